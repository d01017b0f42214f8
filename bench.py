#!/usr/bin/env python3
"""Decode and prefill throughput at Qwen3-8B layer sizes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--shape 8b|0.6b|32b] [--impl ours|reference]
    python bench.py --workload mixed [--shape 0.6b|8b]     # 64 requests, continuous batching
    python bench.py --kernels                               # single kernels at serving sizes
    python bench.py --kernels --attn 16,8,64                # the attention kernels at another head layout
    python bench.py --ablate                                # a decode step with one kind of kernel left out at a time

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 and the context length
of the configuration (a "step" is one decode step of the whole batch), timed on the device with
CUDA events around exactly K steps; ``e2e`` is the same through the Python entry point
(``Engine.step``: host token ids in through pinned memory every step, sampled ids read back every
step).  ``prefill`` times one step of 2,048 prompt tokens; ``roofline`` divides the bytes a decode
step must read (every weight once, the cache of the live requests) by its time; ``points`` holds
decode at batch 1 and 64 at the same context, and ``baseline_b1/8/64``: decode tokens per second
over 256 steps after a 2,048-token prompt (context 2,048 -> 2,304).  Fractions are given against the
measured peaks (MEASURED_PEAKS.json beside this file, when present) and, as ``frac_nominal``, against
the nominal 8 TB/s and 2.25 PFLOP/s.  The logits of the first prefill and of the last decode step
are checked to be finite (their largest magnitudes stand in ``config``).

``--workload mixed``: 64 requests with prompt lengths uniform in 16..2,048 (seeded), 256 new tokens
each, through ``Engine.generate_sync``: decoded and total tokens per second, steps, the distribution
of step times and the number of preemptions, as one JSON line (the reference's batch test,
src/main.rs:103-115, 502-555, is the counterpart).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the headline configuration (Qwen3-8B shape).
CONFIG = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
    tie_word_embeddings=False, sliding_window=None,
)
# The other two published shapes, for --shape: what differs from the headline configuration.
SHAPES = {
    "8b": {},
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 tie_word_embeddings=True),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0
PAGE = 16
SETTLE = 24   # untimed decode steps between a prefill burst and any timed decode step, beside --warmup


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        mhz, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for t, line in self.samples:
            if t < t0 or t > t1 + 0.2:
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                mhz.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Rust crate (no setup.py/pyproject.toml; pip: 'not installable'); "
                      "no Rust toolchain and no network on this machine"}))
    return 0


def check_finite(logits, what: str) -> float:
    """A benchmark line must not come from a model that computes nonsense: every logit finite, and
    not all of them alike.  Returns the largest magnitude."""
    import torch
    v = logits.float()
    if not bool(torch.isfinite(v).all()):
        raise SystemExit(f"bench.py: the logits of {what} are not finite")
    if float(v.max() - v.min()) == 0.0:
        raise SystemExit(f"bench.py: the logits of {what} are all equal")
    return round(float(v.abs().max()), 3)


def mixed_workload(args, cfg, full, pk) -> int:
    """Continuous batching: ``--requests`` requests, prompt lengths uniform in [16, 2048] (seeded), 256 new
    tokens each, greedy, through the Python entry point.  One untimed pass (graphs are captured, buffers
    sized), then the timed one with fresh prompts of the same lengths."""
    import numpy as np
    import torch
    from xinfer_b200.config import EngineConfig
    from xinfer_b200.engine.llm import Engine
    from xinfer_b200.engine.runner import ModelRunner
    from xinfer_b200.sampling import SamplingParams

    N, new_tokens = args.requests, 256
    max_len = 2048 + new_tokens + 64
    runner = ModelRunner.random(cfg, seed=0, dtype="bfloat16", block_size=PAGE, num_blocks=N * (max_len // PAGE + 1),
                                max_num_seqs=N, max_model_len=max_len)
    engine = Engine(EngineConfig(weight_path="(random)", block_size=PAGE, max_num_seqs=N, max_num_batched_tokens=8192,
                                 prefill_chunk_size=2048, max_model_len=max_len, disable_cuda_graph=args.no_graph),
                    "bf16", runner=runner)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    lens = rng.integers(16, 2049, size=N)
    sp = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
    clocks = ClockSampler()
    clocks.start()
    result = None
    for timed in (False, True):
        prompts = [rng.integers(0, V, size=int(n)).tolist() for n in lens]
        before = dict(engine.stats)
        torch.cuda.synchronize()
        t0 = time.time()
        ids = [engine.add_request(p, sp) for p in prompts]
        step_ms = []
        last = t0
        while any(i in engine._live for i in ids):
            engine.step()
            now = time.time()
            step_ms.append((now - last) * 1e3)
            last = now
        torch.cuda.synchronize()
        t1 = time.time()
        outs = [engine._done.pop(i) for i in ids]
        if any(o.error for o in outs) or any(o.decoded_length != new_tokens for o in outs):
            raise SystemExit("bench.py: the mixed workload did not finish every request")
        if timed:
            st = {k: engine.stats[k] - before[k] for k in before}
            decoded, prompt = sum(o.decoded_length for o in outs), int(lens.sum())
            step_ms.sort()
            pick = lambda q: round(step_ms[min(len(step_ms) - 1, int(q * len(step_ms)))], 3)
            result = {
                "metric": f"decoded tok/s, continuous batching of {N} requests (Qwen3-{args.shape.upper()} shape)",
                "value": round(decoded / (t1 - t0), 1), "unit": "tokens/s", "total_tok_s": round((decoded + prompt) / (t1 - t0), 1),
                "n_gpus": 1, "seconds": round(t1 - t0, 3), "steps": st["steps"], "steps_decided_ahead": st["steps_decided_ahead"],
                "preemptions": st["preemptions"], "step_ms": {"p50": pick(0.5), "p90": pick(0.9), "p99": pick(0.99), "max": round(step_ms[-1], 3)},
                "prompt_tokens": prompt, "decoded_tokens": decoded, "dtype": "bf16", "impl": "ours",
                "data": "synthetic (random weights, seeded uniform token ids)", "higher_is_better": True,
                "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": cfg["num_hidden_layers"],
                           "layers_of_config": full["num_hidden_layers"], "requests": N, "prompt_len": "uniform 16..2048",
                           "new_tokens": new_tokens, "page_size": PAGE, "max_num_batched_tokens": 8192,
                           "prefill_chunk_size": 2048, "cuda_graph": not args.no_graph},
                "clocks": clocks.summary(t0, t1),
            }
    clocks.stop()
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES),
                    help="layer sizes: the headline Qwen3-8B shape (default) or the 0.6B / 32B shapes")
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (reported in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--workload", default="steps", choices=["steps", "mixed"],
                    help="'mixed': 64 requests of 16..2,048 prompt tokens under continuous batching, instead of the step benchmark")
    ap.add_argument("--requests", type=int, default=64, help="requests of the mixed workload")
    ap.add_argument("--ablate", action="store_true",
                    help="instead of the step benchmark: a decode step with one kind of kernel left out at a time (what each kind costs in the chain)")
    ap.add_argument("--attn", default="", metavar="HEADS,KV_HEADS,HEAD_DIM[,PAGE_SIZE]",
                    help="with --kernels: the attention kernels alone at this head layout, over short and long contexts")
    ap.add_argument("--case", default="", metavar="decode:BATCHxCONTEXT | prefill:CACHED+NEW",
                    help="with --kernels --attn: this one case instead of the standard ones")
    ap.add_argument("--kernels", action="store_true",
                    help="instead of the step benchmark, time single kernels at serving sizes: one JSON line each")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)
    if args.ablate:
        from xinfer_b200 import measure
        for rec in measure.decode_ablation(dict(CONFIG, **SHAPES[args.shape]), layers=args.layers or 12):
            print(json.dumps(rec), flush=True)
        return 0
    if args.kernels and args.attn:
        # the attention kernels alone at another head layout: HEADS,KV_HEADS,HEAD_DIM[,PAGE_SIZE]
        from xinfer_b200 import measure
        pk = peaks()
        sizes = [int(x) for x in args.attn.split(",")]
        lay = dict(heads=sizes[0], kv_heads=sizes[1], head_dim=sizes[2], page_size=sizes[3] if len(sizes) > 3 else PAGE)
        decode_cases, prefill_cases = ((1, 4096), (8, 4096), (64, 2048), (4, 65536), (16, 512)), ((0, 512), (0, 2048), (0, 8192), (30000, 2048))
        if args.case:      # one case alone (its first launch is a plain one: what a profiler is pointed at)
            kind, _, size = args.case.partition(":")
            if kind == "decode":
                decode_cases, prefill_cases = (tuple(int(x) for x in size.split("x")),), ()
            elif kind == "prefill":
                decode_cases, prefill_cases = (), (tuple(int(x) for x in size.split("+")),)
            else:
                raise SystemExit("bench.py: --case is decode:BATCHxCONTEXT or prefill:CACHED+NEW")
        for rec in (measure.decode_attention(decode_cases, hbm_gbs=pk["hbm_gbs"], **lay)
                    + measure.prefill_attention(prefill_cases, peak_tflops=pk["bf16_tflops"], **lay)):
            print(json.dumps(dict(rec, **lay)), flush=True)
        return 0
    if args.kernels:
        from xinfer_b200 import measure
        pk = peaks()
        for rec in (measure.decode_gemms(hbm_gbs=pk["hbm_gbs"]) + measure.decode_attention(hbm_gbs=pk["hbm_gbs"])
                    + measure.prefill_attention(peak_tflops=pk["bf16_tflops"]) + measure.prefill_elementwise(hbm_gbs=pk["hbm_gbs"])
                    + measure.sampling()):
            print(json.dumps(rec), flush=True)
        return 0

    import numpy as np
    import torch
    from xinfer_b200 import kernels
    from xinfer_b200.config import EngineConfig
    from xinfer_b200.engine.llm import Engine
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.sampling import SamplingParams

    pk = peaks()
    full = dict(CONFIG, **SHAPES[args.shape])
    cfg = dict(full, num_hidden_layers=args.layers or full["num_hidden_layers"])
    if args.workload == "mixed":
        return mixed_workload(args, cfg, full, pk)
    max_b = args.batch if args.no_points else max(args.batch, 64)
    if args.context < 256:
        raise SystemExit("bench.py: --context must be at least 256")
    longest = max(args.context, PREFILL_TOKENS + 256)     # the prefill measurement and the reference's decode setting need their room
    pages_per_req = (longest + PAGE - 1) // PAGE + 1
    t_load = time.time()
    runner = ModelRunner.random(cfg, seed=0, dtype="bfloat16", block_size=PAGE, num_blocks=max_b * pages_per_req,
                                max_num_seqs=max_b, max_model_len=longest + 64)
    torch.cuda.synchronize()
    load_s = time.time() - t_load
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    use_graph = not args.no_graph

    def fill(batch: int, ctx: int):
        """Open `batch` requests and prefill each to `ctx` tokens through the step function."""
        slots = [runner.open_request() for _ in range(batch)]
        chunk = 4096
        for s in slots:
            at = 0
            while at < ctx:
                n = min(chunk, ctx - at)
                runner.step([StepInput(s, rng.integers(0, V, size=n), [])])
                at += n
        runner.check_errors()
        return slots

    def decode_device(slots, n_steps: int, n_warm: int):
        """K decode steps, kernel time only: token ids come from the host each step, no read-back."""
        n_warm += SETTLE   # the prefill before leaves the device at its power cap: untimed steps until the clocks are back
        toks = rng.integers(0, V, size=(n_steps + n_warm, len(slots)))
        for i in range(n_warm):
            runner.step([StepInput(s, toks[i, j:j + 1], [0]) for j, s in enumerate(slots)], allow_graph=use_graph)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches = 0
        t0 = time.time()
        e0.record()
        for i in range(n_warm, n_warm + n_steps):
            runner.step([StepInput(s, toks[i, j:j + 1], [0]) for j, s in enumerate(slots)], allow_graph=use_graph)
            launches += runner.last_launches
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        runner.check_errors()
        return e0.elapsed_time(e1) / n_steps, launches, (t0, t1)

    def close(slots):
        for s in slots:
            runner.close_request(s)

    clocks = ClockSampler()
    clocks.start()

    # ---- prefill: one step of 2,048 prompt tokens ------------------------------------------------------
    pre_ms = []
    for i in range(3 + 3):
        s = runner.open_request()
        ids = rng.integers(0, V, size=PREFILL_TOKENS)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = runner.step([StepInput(s, ids, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if i == 0:
            absmax_prefill = check_finite(logits, "the first prefill")
        if i >= 3:
            pre_ms.append(e0.elapsed_time(e1))
        runner.close_request(s)
    runner.check_errors()
    pre = min(pre_ms)
    L, H, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_params = H * (nh + 2 * nkv) * d + nh * d * H + 3 * H * I
    T = PREFILL_TOKENS
    flops = 2.0 * T * layer_params * L + 2.0 * V * H + L * 4.0 * nh * d * (T * (T + 1) / 2)
    prefill = {"value": round(T / (pre / 1e3), 1), "tokens": T, "ms": round(pre, 3),
               "frac": round(flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_nominal": round(flops / (pre / 1e3) / (NOMINAL_BF16_TFLOPS * 1e12), 4)}

    # ---- decode at the headline batch --------------------------------------------------------------------
    B = args.batch
    ctx0 = args.context - steps - warmup - SETTLE - 2
    if ctx0 < 16:
        raise SystemExit(f"bench.py: --steps {steps} with --warmup {warmup} does not fit a context of {args.context} "
                         f"(the timed steps end at the context length): give a larger --context or fewer steps")
    slots = fill(B, ctx0)
    ms, launches, (t0, t1) = decode_device(slots, steps, warmup)
    ck = clocks.summary(t0, t1)
    value = B / (ms / 1e3)
    weight_bytes = (layer_params * L + V * H) * 2 + (2 * L + 1) * H * 4 + L * 2 * d * 4
    ctx_mid = ctx0 + warmup + SETTLE + steps / 2
    kv_bytes = runner.kv_bytes_per_token * ctx_mid * B
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "frac_nominal": round(achieved / NOMINAL_HBM_GBS, 4)}
    absmax_decode = check_finite(runner.step([StepInput(s, rng.integers(0, V, size=1), [0]) for s in slots],
                                             allow_graph=use_graph), "the last decode step")
    close(slots)

    # ---- the same through the Python entry point ----------------------------------------------------------
    econfig = EngineConfig(weight_path="(random)", block_size=PAGE, max_num_seqs=max_b, max_num_batched_tokens=8192,
                           prefill_chunk_size=4096, max_model_len=longest + 64, disable_cuda_graph=not use_graph)
    engine = Engine(econfig, "bf16", runner=runner)
    n_e2e = min(steps, 64)
    # prompts are prefilled two per step, so requests start decoding a few steps apart: leave room
    # for that in the context, and let no request finish inside the timed region
    # the prompts' prefill leaves the device at its power cap for some tens of milliseconds: decode steps
    # run untimed until the clocks have come back
    e2e_warmup = warmup + SETTLE
    margin = B // 2 + 8
    prompt_len = args.context - n_e2e - e2e_warmup - margin - 8     # prompt + max_tokens stays inside a request's pages
    sp = SamplingParams(temperature=0.0, max_tokens=n_e2e + e2e_warmup + margin, ignore_eos=True)
    for _ in range(B):
        engine.add_request(rng.integers(0, V, size=prompt_len).tolist(), sp)
    while any(engine.scheduler.output(i) == [] for i in list(engine._live)):   # prompts, first tokens
        engine.step()
    for _ in range(e2e_warmup):
        engine.step()
    # The clock runs from one step's tokens reaching the host to those of the n-th step after it.  The
    # engine queues the next step before it waits for the current one, so the device is never drained
    # here: a synchronisation at the start would let the first timed call find its step already done.
    tw0 = time.time()
    done_before = engine.stats["decoded_tokens"]
    h2d = 0
    for _ in range(n_e2e):
        engine.step()   # returns when this step's tokens are on the host (the next step is already queued)
        h2d += runner.assembler.h2d_bytes + B * kernels.SAMPLE_PARAMS.itemsize
    tw1 = time.time()
    torch.cuda.synchronize()
    e2e_tokens = engine.stats["decoded_tokens"] - done_before
    e2e = {"value": round(e2e_tokens / (tw1 - tw0), 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d // n_e2e,
           "d2h_bytes_per_step": B * 4 + 4}
    for seq_id in list(engine._live):   # the timed steps are done: drop what is still running
        engine.scheduler.abort(seq_id)
    while engine.has_work():
        engine.step()
    for seq_id in engine.scheduler.drain_finished():
        engine._finish(seq_id)

    # ---- batch 1 and 64 -----------------------------------------------------------------------------------
    points = {}
    if not args.no_points:
        for b in (1, 64):
            k = min(steps, 32)
            sl = fill(b, args.context - k - warmup - SETTLE - 2)
            m, _, _ = decode_device(sl, k, warmup)
            points[f"decode_b{b}"] = round(b / (m / 1e3), 1)
            close(sl)
        # the reference configuration's own decode setting: a 2,048-token prompt, then 256 decoded tokens
        for b in (1, 8, 64):
            sl = fill(b, PREFILL_TOKENS - warmup - SETTLE)
            m, _, _ = decode_device(sl, 256, warmup)
            points[f"baseline_b{b}"] = round(b / (m / 1e3), 1)
            close(sl)
    clocks.stop()

    out = {
        "metric": f"decode tok/s at batch {B} (Qwen3-{args.shape.upper()} shape, context {args.context})", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, seeded uniform token ids)",
        "impl": "ours",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": cfg["num_hidden_layers"], "layers_of_config": full["num_hidden_layers"],
                   "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V,
                   "global_batch": B, "seq_len": args.context, "page_size": PAGE, "parallelism": "1 GPU",
                   "cuda_graph": use_graph, "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": pk["source"], "settle_steps": SETTLE,
                   "logit_absmax_prefill": absmax_prefill, "logit_absmax_decode": absmax_decode},
        "clocks": ck, "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill, "roofline": roofline, "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
