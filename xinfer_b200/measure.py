"""Timings of single kernels at serving sizes, with CUDA events, for ``bench.py --kernels``.

Each function returns a list of records (dicts); times are medians over repeated launches.  Decode
kernels are timed inside a CUDA graph of several launches over different data (larger than the
L2), the way a decode step runs them; prefill attention is replayed from a graph of a few launches.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, List, Sequence

import numpy as np
import torch

from . import kernels
from .parts import LayerCache, Workspace
from .parts import attention_backend


def _graph_time_us(run, per: int, repeats: int = 8) -> float:
    """Median time of one of the ``per`` launches that ``run`` makes, replayed from a CUDA graph."""
    torch.cuda.synchronize()   # what the caller prepared on the current stream is done
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0 / per)
    return float(sorted(times)[len(times) // 2])


def _attention_context(entries, page_size: int, device):
    """Step metadata for `entries` = [(cached tokens, new tokens)], pages handed out in shuffled order."""
    to = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=device)
    counts = [c for _, c in entries]
    q_start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    pages_per = max((s + c + page_size - 1) // page_size for s, c in entries)
    num_pages = len(entries) * pages_per + 1
    table = np.random.default_rng(0).permutation(num_pages - 1)[: len(entries) * pages_per].reshape(len(entries), pages_per)
    pos = np.concatenate([np.arange(s, s + c) for s, c in entries])
    req = np.concatenate([np.full(c, b) for b, (_, c) in enumerate(entries)])
    ctx = SimpleNamespace(
        positions=to(pos), req_of_token=to(req), q_start=to(q_start), start_pos=to([s for s, _ in entries]),
        num_entries=len(entries), num_tokens=int(q_start[-1]), h_q_start=q_start, real_entries=len(entries),
        h_start_pos=np.asarray([s for s, _ in entries], dtype=np.int32), max_context=max(s + c for s, c in entries),
        fixed_shapes=False, scratch={}, workspace=Workspace(device), err=torch.zeros(1, dtype=torch.int32, device=device))
    return ctx, to(table.astype(np.int32)), pages_per, num_pages


def decode_attention(cases: Sequence = ((1, 4096), (8, 4096), (64, 4096), (8, 32768)), *, heads: int = 32,
                     kv_heads: int = 8, head_dim: int = 128, page_size: int = 16, hbm_gbs: float = 0.0,
                     device="cuda:0") -> List[Dict]:
    """One decode token per request over `context` cached tokens, for (batch, context) cases."""
    out = []
    for batch, context in cases:
        ctx, table, stride, num_pages = _attention_context([(context - 1, 1)] * batch, page_size, device)
        layers = 8 if batch * context <= 8 * 32768 else 2
        caches = [LayerCache.of_keys_and_values(torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(),
                             torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(), 0, page_size)
                  for _ in range(layers)]
        q = torch.randn(batch, heads, head_dim, device=device).bfloat16()
        o = torch.empty_like(q)
        nbytes = batch * context * kv_heads * head_dim * 2 * 2
        rec = {"kernel": "decode attention", "batch": batch, "context": context, "bytes": nbytes}
        for name, flag in (("tcgen05_us", True), ("mma_sync_us", False)):
            attention_backend.DECODE_TC = flag
            try:
                # as in a step: the work is planned once, before the first kernel, for all layers
                ctx.scratch.clear()
                attention_backend.prepare_step(ctx, torch.bfloat16, heads, kv_heads, head_dim, page_size, None, stride)
                torch.cuda.synchronize()   # the launches below run on a stream of their own
                rec[name] = round(_graph_time_us(lambda: [attention_backend.attend(o, q, c, ctx, table, stride, None, head_dim ** -0.5)
                                                          for c in caches], layers), 1)
            finally:
                attention_backend.DECODE_TC = True
        if int(ctx.err):
            raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(ctx.err)))
        rec["gbs"] = round(nbytes / rec["tcgen05_us"] / 1e3, 1)
        if hbm_gbs:
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_gbs, 3)
        out.append(rec)
    return out


def prefill_attention(cases: Sequence = ((0, 2048), (0, 8192), (24576, 8192)), *, heads: int = 32, kv_heads: int = 8,
                      head_dim: int = 128, page_size: int = 16, peak_tflops: float = 0.0, device="cuda:0") -> List[Dict]:
    """One request bringing `new` tokens after `cached` ones, for (cached, new) cases."""
    out = []
    for cached, new in cases:
        ctx, table, stride, num_pages = _attention_context([(cached, new)], page_size, device)
        cache = LayerCache.of_keys_and_values(torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(),
                           torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(), 0, page_size)
        q = torch.randn(new, heads, head_dim, device=device).bfloat16()
        o = torch.empty_like(q)
        flops = 4.0 * heads * head_dim * (new * cached + new * (new + 1) / 2)
        rec = {"kernel": "prefill attention", "cached": cached, "new": new, "flops": flops}
        for name, flag in (("tcgen05_us", True), ("mma_sync_us", False)):
            attention_backend.PREFILL_TC = flag
            try:
                # several launches replayed from a CUDA graph: the host's share of a launch (tensor maps, wrappers)
                # is not in the time, as it is not in a step, where launches queue ahead of the device
                per = 4 if new * (cached + new) <= 8192 * 16384 else 1
                attention_backend.prepare_step(ctx, torch.bfloat16, heads, kv_heads, head_dim, page_size, None, stride)
                torch.cuda.synchronize()
                rec[name] = round(_graph_time_us(lambda: [attention_backend.attend(o, q, cache, ctx, table, stride, None, head_dim ** -0.5)
                                                          for _ in range(per)], per), 1)
            finally:
                attention_backend.PREFILL_TC = True
        if int(ctx.err):
            raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(ctx.err)))
        rec["tflops"] = round(flops / rec["tcgen05_us"] / 1e6, 1)
        if peak_tflops:
            rec["frac_of_peak"] = round(rec["tflops"] / peak_tflops, 3)
        out.append(rec)
    return out


def decode_gemms(tokens: Sequence[int] = (1, 8, 32), *, hidden: int = 4096, heads: int = 32, kv_heads: int = 8,
                 head_dim: int = 128, intermediate: int = 12288, hbm_gbs: float = 0.0, device="cuda:0") -> List[Dict]:
    """The four matrix products of a layer, one after the other as in a decode step, for M tokens:
    the streaming tcgen05 kernel and the library product."""
    shapes = [((heads + 2 * kv_heads) * head_dim, hidden), (hidden, heads * head_dim), (2 * intermediate, hidden),
              (hidden, intermediate)]
    layer_bytes = sum(n * k * 2 for n, k in shapes)
    layers = max(2, int(600e6 / layer_bytes) + 1)      # more weights than the L2 holds
    ws = [[(torch.randn(n, k, device=device) * 0.02).bfloat16() for n, k in shapes] for _ in range(layers)]
    err = torch.zeros(1, dtype=torch.int32, device=device)
    out = []
    for m in tokens:
        xs = {k: torch.randn(m, k, device=device).bfloat16() for _, k in shapes}
        ys = {n: torch.empty(m, n, dtype=torch.bfloat16, device=device) for n, _ in shapes}

        def own():
            for l in range(layers):
                for (n, k), w in zip(shapes, ws[l]):
                    if not kernels.gemm_skinny_tc(ys[n], xs[k], w, err):
                        raise RuntimeError(f"the streaming kernel does not take M={m}, N={n}, K={k}")

        def lib():
            for l in range(layers):
                for (n, k), w in zip(shapes, ws[l]):
                    torch.mm(xs[k], w.t(), out=ys[n])

        rec = {"kernel": "decode matrix products of a layer", "tokens": m, "bytes": layer_bytes,
               "tcgen05_us": round(_graph_time_us(own, layers), 1), "library_us": round(_graph_time_us(lib, layers), 1)}
        rec["gbs"] = round(layer_bytes / rec["tcgen05_us"] / 1e3, 1)
        if hbm_gbs:
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_gbs, 3)
        out.append(rec)
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def _loop_time_us(run, repeats: int = 9) -> float:
    """Median time of one call of ``run`` (CUDA events, a synchronisation on both sides)."""
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0)
    return float(sorted(times)[len(times) // 2])


def prefill_elementwise(tokens: int = 2048, *, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, head_dim: int = 128,
                        intermediate: int = 12288, page_size: int = 16, hbm_gbs: float = 0.0, device="cuda:0") -> List[Dict]:
    """The memory-bound kernels between the matrix products at a prompt portion's size: residual sum +
    RMSNorm, q/k norm + rotation + cache write, SiLU gate.  Each call works on one of several sets of
    buffers in turn, together larger than the L2, and the time is per call."""
    sets = 4
    err = torch.zeros(1, dtype=torch.int32, device=device)
    bf = lambda *shape: torch.randn(*shape, device=device).bfloat16()
    out = []

    def record(name, nbytes, run):
        us = _loop_time_us(lambda: [run(i) for i in range(sets)]) / sets
        rec = {"kernel": name, "tokens": tokens, "bytes": nbytes, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
        if hbm_gbs:
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_gbs, 3)
        out.append(rec)

    # residual sum + RMSNorm: reads x and the branch, writes the sum and the normed rows
    xs, bs, os_ = [bf(tokens, hidden) for _ in range(sets)], [bf(tokens, hidden) for _ in range(sets)], [bf(tokens, hidden) for _ in range(sets)]
    w = torch.randn(hidden, device=device).float()
    record("residual sum + RMSNorm", 4 * tokens * hidden * 2,
           lambda i: kernels.rmsnorm(os_[i], xs[i], w, 1e-6, err, branch=bs[i], sum_out=xs[i]))
    # q/k norm + rotation + cache write: reads the packed projection, writes q and the pages
    width = (heads + 2 * kv_heads) * head_dim
    qkvs = [bf(tokens, width) for _ in range(sets)]
    qs = [torch.empty(tokens, heads, head_dim, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    pages = (tokens + page_size - 1) // page_size
    kc = [torch.zeros(pages, kv_heads, page_size, head_dim, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    vc = [torch.zeros_like(k) for k in kc]
    qw, kw = torch.randn(head_dim, device=device).float(), torch.randn(head_dim, device=device).float()
    half = head_dim // 2
    cos, sin = torch.randn(tokens, half, device=device).float(), torch.randn(tokens, half, device=device).float()
    pos = torch.arange(tokens, dtype=torch.int32, device=device)
    req = torch.zeros(tokens, dtype=torch.int32, device=device)
    table = torch.randperm(pages, device=device).to(torch.int32)
    record("q/k norm + rotation + cache write", 2 * tokens * width * 2,
           lambda i: kernels.qk_norm_rope_write(qs[i], kc[i], vc[i], qkvs[i], qw, kw, cos, sin, pos, req, table, pages, heads, kv_heads,
                                                head_dim, head_dim, False, 1e-6, True, err))
    # SiLU gate: reads gate and up, writes their product
    gus = [bf(tokens, 2 * intermediate) for _ in range(sets)]
    acts = [torch.empty(tokens, intermediate, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    record("SiLU gate", 3 * tokens * intermediate * 2, lambda i: kernels.swiglu(acts[i], gus[i]))
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def sampling(rows: Sequence[int] = (1, 8, 64), *, vocab: int = 151936, device="cuda:0") -> List[Dict]:
    """The sampling kernel alone (no host work, no copies) over float32 logits, per way of sampling."""
    from .sampling import SamplingParams
    from .sampling.sampler import Sampler
    ways = (("greedy", SamplingParams(temperature=0.0)), ("temperature", SamplingParams(temperature=0.8)),
            ("top-k 20, top-p 0.95", SamplingParams(temperature=0.6, top_k=20, top_p=0.95)),
            ("top-p 0.9", SamplingParams(temperature=0.8, top_p=0.9)), ("top-k 1000", SamplingParams(temperature=0.8, top_k=1000)))
    out = []
    for r in rows:
        logits = torch.randn(r, vocab, device=device) * 3
        s = Sampler(device, r)
        rec = {"kernel": "sampling", "rows": r, "vocab": vocab}
        for name, sp in ways:
            s.sample(logits, [sp] * r, [1] * r, [0] * r, None)     # leaves the rows' parameters on the device
            rec[name + " us"] = round(_graph_time_us(lambda: [kernels.sample(s._out_dev, logits, s._params_dev, s._hist_dev, False,
                                                                             s._scratch, None, capacity=r) for _ in range(8)], 8), 1)
        out.append(rec)
    return out


def decode_ablation(config: Dict, *, layers: int = 12, batches: Sequence[int] = (1, 8), context: int = 3900,
                    page_size: int = 16, device="cuda:0") -> List[Dict]:
    """What each kind of kernel costs IN the chain of a decode step: the step is timed whole and with one
    kind of kernel left out (the numbers it computes are then wrong; its launches are gone, everything
    else is as in the product: CUDA graph, programmatic dependent launch).  The difference is what
    that kind really costs, start-up and drain included and whatever it hides of its neighbours
    excluded; beside it stands what its bytes would take at the measured copy rate."""
    from .engine.runner import ModelRunner, StepInput
    from .parts import attention as attention_part
    from .parts import attention_backend as backend
    from .parts import norm as norm_part
    from .parts import swiglu as swiglu_part

    cfg = dict(config, num_hidden_layers=layers)
    rng = np.random.default_rng(0)

    def timed(batch: int) -> float:
        runner = ModelRunner.random(cfg, seed=0, dtype="bfloat16", block_size=page_size, device=device,
                                    num_blocks=batch * (context // page_size + 20), max_num_seqs=batch, max_model_len=context + 256)
        slots = [runner.open_request() for _ in range(batch)]
        for s in slots:
            runner.step([StepInput(s, rng.integers(0, 1000, size=context), [])])
        one = lambda: runner.step([StepInput(s, rng.integers(0, 1000, size=1), [0]) for s in slots], allow_graph=True)
        for _ in range(30):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(64):
            one()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 64 * 1000.0

    keep = (kernels.swiglu, kernels.qk_norm_rope_write, backend.attend, attention_part.linear, swiglu_part.linear,
            norm_part.RMSNorm.forward)

    def no_norm(self, out, x, ctx, branch=None, sum_out=None, rows=None):
        return keep[5](self, out, x, ctx, branch, sum_out, rows) if rows is not None else out

    variants = [
        ("whole step", lambda: None),
        ("norms (two per layer)", lambda: setattr(norm_part.RMSNorm, "forward", no_norm)),
        ("q/k norm + rotation + cache write", lambda: setattr(kernels, "qk_norm_rope_write", lambda *a, **k: None)),
        ("attention", lambda: setattr(backend, "attend", lambda *a, **k: None)),
        ("q/k/v and output products", lambda: setattr(attention_part, "linear", lambda out, x, w, err=None: out)),
        ("SiLU gate", lambda: setattr(kernels, "swiglu", lambda out, gu: None)),
        ("gate/up and down products", lambda: setattr(swiglu_part, "linear", lambda out, x, w, err=None: out)),
    ]
    out = []
    try:
        for batch in batches:
            whole = None
            for name, patch in variants:
                patch()
                try:
                    us = timed(batch)
                finally:
                    (kernels.swiglu, kernels.qk_norm_rope_write, backend.attend, attention_part.linear, swiglu_part.linear) = keep[:5]
                    norm_part.RMSNorm.forward = keep[5]
                if whole is None:
                    whole = us
                    out.append({"kernel": "decode step", "batch": batch, "layers": layers, "us_per_step": round(us, 1)})
                else:
                    out.append({"kernel": "decode step without " + name, "batch": batch, "us_per_step": round(us, 1),
                                "cost_in_chain_us_per_layer": round((whole - us) / layers, 1)})
    finally:
        (kernels.swiglu, kernels.qk_norm_rope_write, backend.attend, attention_part.linear, swiglu_part.linear) = keep[:5]
        norm_part.RMSNorm.forward = keep[5]
    return out
