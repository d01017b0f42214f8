"""The model runner: owns the model, the cache manager with its device pages, per-request state
and the ONE step function everything else drives (generation, trace replay, the benchmark).

``step(entries)`` takes a batch of (request slot, its next tokens, wanted positions): portions of
prompts beside single decoded tokens, cut anywhere.  It takes the pages those tokens need, runs
only those tokens as one batch against the cache and returns float32 logits at the wanted
positions.  The reference's counterpart is ``ModelRunner::run`` (src/core/runner.rs:1018), which
runs either prompt chunks or decode tokens, never both, and returns sampled ids
(prepare_prefill :1303-1563, prepare_decode :1565-1750).

Steps in which every request brings exactly one token and wants its logits may be replayed from a
CUDA graph (one per padded batch size and block-table width), as the reference captures its
decode step per batch size (src/utils/graph.rs:400-420, 689-711).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels, tracing
from ..cache.manager import CacheGroup, CacheManager, StateSlots
from ..config import ConfigError, config_from_dict, load_config
from ..models.decoder import DecoderModel, model_weight_specs
from ..native import host_lib
from ..parts import LayerCache, StepContext, Workspace
from ..weights.loader import WeightStore


class StepError(RuntimeError):
    pass


@dataclass
class StepInput:
    slot: int                 # the request's slot, from ``open_request``
    tokens: Sequence[int]     # its next tokens (a prompt portion, or one decoded token)
    want: Sequence[int] = ()  # positions among these tokens whose logits are wanted


def _dtype_of(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.float32, torch.bfloat16):
            return name
        raise ConfigError(f"dtype {name} is not supported (bfloat16 or float32)")
    key = str(name).lower()
    if key in ("bf16", "bfloat16"):
        return torch.bfloat16
    if key in ("f32", "fp32", "float32"):
        return torch.float32
    raise ConfigError(f"dtype '{name}' is not supported (bf16/bfloat16 or f32/float32)")


def resolve_max_model_len(asked: Optional[int], max_positions: int) -> int:
    """The longest sequence the engine will hold: what was asked for, or all positions the model's
    position tables have.  More than the tables hold is refused here, before any token could run
    at a position without an angle."""
    if asked is None:
        return int(max_positions)
    asked = int(asked)
    if asked <= 0:
        raise ConfigError(f"max_model_len must be positive, got {asked}")
    if asked > max_positions:
        raise ConfigError(f"max_model_len {asked} exceeds the model's max_position_embeddings {max_positions}: "
                          f"its position tables end there")
    return asked


class _MetaBuffers:
    """A small ring of pinned staging buffers with a device twin each; a buffer is reused only
    after the copy that read it has finished."""

    def __init__(self, device, depth: int = 3):
        self.device = device
        self.depth = depth
        self.cap = 0
        self.host: List[torch.Tensor] = []
        self.dev: List[torch.Tensor] = []
        self.events: List[Optional[torch.cuda.Event]] = []
        self.i = 0

    def reserve(self, n: int) -> None:
        if n <= self.cap:
            return
        torch.cuda.synchronize(self.device)
        self.cap = max(n, 2 * self.cap, 4096)
        self.host = [torch.empty(self.cap, dtype=torch.int32, pin_memory=True) for _ in range(self.depth)]
        self.dev = [torch.empty(self.cap, dtype=torch.int32, device=self.device) for _ in range(self.depth)]
        self.events = [None] * self.depth

    def next(self) -> Tuple[torch.Tensor, torch.Tensor, int]:
        self.i = (self.i + 1) % self.depth
        ev = self.events[self.i]
        if ev is not None:
            ev.synchronize()
        return self.host[self.i], self.dev[self.i], self.i

    def sent(self, i: int) -> None:
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class StepAssembler:
    """Turns a batch of ``StepInput`` into a ``StepContext``: takes the pages the tokens need,
    packs the step's metadata natively into a pinned buffer and sends it with one copy."""

    def __init__(self, cache: CacheManager, *, vocab_size: int, max_model_len: int, dtype: torch.dtype,
                 device, workspace: Optional[Workspace] = None, err: Optional[torch.Tensor] = None):
        self.cache = cache
        self.vocab_size = int(vocab_size)
        self.max_model_len = int(max_model_len)
        self.dtype = dtype
        self.device = torch.device(device)
        self.page_sizes = [g.page_size for g in cache.groups]
        self.workspace = workspace if workspace is not None else Workspace(self.device)
        self.err = err if err is not None else torch.zeros(1, dtype=torch.int32, device=self.device)
        self._meta = _MetaBuffers(self.device)
        self._lib = host_lib()
        self.h2d_bytes = 0   # bytes of the last step's metadata copy
        # ids a sampler left on the device: a token id -1 - i of a step stands for sampled[i]
        self.sampled: Optional[torch.Tensor] = None

    def prepare(self, entries: Sequence[StepInput], *, pad_entries: int = 0, pad_tokens: int = 0,
                pad_rows: int = 0, strides: Optional[Sequence[int]] = None,
                into: Optional[torch.Tensor] = None, workspace: Optional[Workspace] = None) -> StepContext:
        """``into``: a device buffer that must receive the metadata (a CUDA graph reads it at a
        fixed address); otherwise a buffer of the ring is used."""
        if not entries:
            raise StepError("a step needs at least one entry")
        B = len(entries)
        counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=B)
        if (counts <= 0).any():
            raise StepError("every entry of a step must bring at least one token")
        slots = np.fromiter((e.slot for e in entries), dtype=np.int32, count=B)
        if len(set(slots.tolist())) != B:
            raise StepError("a request may appear only once in a step")
        T = int(counts.sum())
        tokens = np.empty(T, dtype=np.int32)
        want_e: List[int] = []
        want_o: List[int] = []
        t = 0
        V = self.vocab_size
        starts = np.empty(B, dtype=np.int32)
        cache = self.cache
        for b, e in enumerate(entries):
            n = int(counts[b])
            tokens[t:t + n] = e.tokens
            t += n
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"entry {b} wants logits at {w}, but brings {n} tokens")
                want_e.append(b)
                want_o.append(int(w))
            slot = int(slots[b])
            if not cache.is_live(slot):
                raise StepError(f"entry {b}: slot {slot} is not an open request")
            start = cache.length(slot)
            starts[b] = start
            if start + n > self.max_model_len:
                raise StepError(f"entry {b}: {start + n} tokens exceed the longest sequence {self.max_model_len}")
            if not cache.extend(slot, start + n):
                raise StepError(f"entry {b}: the page pool has no room for {n} more tokens "
                                f"(free pages {[cache.free_pages(g) for g in range(len(cache.groups))]})")
        low = -self.sampled.numel() if self.sampled is not None else 0
        if tokens.min() < low or tokens.max() >= V:
            raise StepError(f"token ids must lie in [0, {V}); got {int(tokens.min())}..{int(tokens.max())}")
        R = len(want_e)
        G = len(cache.groups)
        Bp, Tp, Rp = max(B, pad_entries), max(T, pad_tokens), max(R, pad_rows, 1)
        longest = int((starts + counts).max())
        max_stride = max(max((longest + ps - 1) // ps for ps in self.page_sizes) + 8, max(strides) if strides else 0)
        need = 3 * (Tp + 4) + 3 * (Bp + 5) + Rp + 8 + G * (Bp * max_stride + 4) + 64
        self._meta.reserve(need)
        host, dev, which = self._meta.next()
        offs = (ctypes.c_longlong * (7 + 2 * G))()
        we = np.asarray(want_e, dtype=np.int32)
        wo = np.asarray(want_o, dtype=np.int32)
        st = np.asarray(strides, dtype=np.int32) if strides is not None else None
        used = self._lib.xb_assemble(
            cache.handle, B, slots.ctypes.data, counts.ctypes.data, tokens.ctypes.data, R,
            we.ctypes.data if R else None, wo.ctypes.data if R else None, int(pad_tokens), int(pad_entries),
            int(pad_rows), st.ctypes.data if st is not None else None, host.data_ptr(), host.numel(), offs)
        if used < 0:
            raise StepError({-1: "step metadata does not fit its buffer", -2: "a slot is not live",
                             -3: "pages are missing for an entry", -4: "a wanted position is out of range"}.get(used, f"assemble failed ({used})"))
        if into is not None:
            if into.numel() < used:
                raise StepError("the graph's metadata buffer is smaller than the step's metadata")
            dev = into
        dev[:used].copy_(host[:used], non_blocking=True)
        self._meta.sent(which)
        self.h2d_bytes = int(used) * 4

        def view(k, n):
            return dev[offs[k]: offs[k] + n]

        return StepContext(
            dtype=self.dtype, device=self.device, num_tokens=Tp, num_entries=Bp,
            token_ids=view(0, Tp), positions=view(1, Tp), req_of_token=view(2, Tp),
            q_start=view(3, Bp + 1), start_pos=view(4, Bp), slots=view(5, Bp),
            logit_rows=view(6, Rp), num_logit_rows=max(R, pad_rows),
            tables=[dev[offs[7 + g]: offs[7 + g] + Bp * offs[7 + G + g]] for g in range(G)],
            strides=[int(offs[7 + G + g]) for g in range(G)],
            err=self.err, workspace=workspace if workspace is not None else self.workspace,
            h_q_start=host[offs[3]: offs[3] + Bp + 1].numpy().copy(), h_start_pos=starts, h_slots=slots,
            real_tokens=T, real_entries=B, max_context=longest, all_single=bool((counts == 1).all()),
            fixed_shapes=into is not None, sampled=self.sampled,
        )


@dataclass
class _DecodeGraph:
    graph: torch.cuda.CUDAGraph
    meta: torch.Tensor          # the device metadata buffer the graph reads
    logits: torch.Tensor        # [bucket, vocab] float32, written by the graph
    launches: int               # kernels of ours inside the graph


def _bucket(n: int, cap: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return min(b, max(cap, n))


class ModelRunner:
    def __init__(self, model_dir: Optional[str], dtype="bfloat16", *, block_size: int = 16,
                 num_blocks: Optional[int] = None, max_num_seqs: int = 32,
                 kv_fraction: float = 0.7, device="cuda:0", max_model_len: Optional[int] = None,
                 model: Optional[DecoderModel] = None, poison_freed_pages: bool = False):
        """``poison_freed_pages`` (debug): every page that goes back to its pool is filled with NaN in
        every layer before the next step runs, so a kernel that read a stale page would show at once."""
        if not torch.cuda.is_available():
            raise StepError("no CUDA device: this engine runs on a B200 (sm_100a) only and has no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        cap = torch.cuda.get_device_capability(self.device)
        if cap[0] != 10:
            raise StepError(f"device {self.device} has compute capability {cap[0]}.{cap[1]}; the kernels are built for sm_100a")
        self.dtype = _dtype_of(dtype)
        kernels.kernels_lib()  # build / load now, loudly
        if model is None:
            entry, cfg = load_config(model_dir)
            model = DecoderModel(entry.plan_of(cfg), self.dtype, self.device)
            store = WeightStore(model_dir)
            try:
                model.load(store)
            finally:
                store.close()
        self.model = model
        self.plan = model.plan
        self.block_size = int(block_size)
        self.max_num_seqs = int(max_num_seqs)
        self.max_model_len = resolve_max_model_len(max_model_len, self.plan.max_positions)
        self.workspace = Workspace(self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._build_caches(num_blocks, kv_fraction)
        self.assembler = StepAssembler(self.cache, vocab_size=self.plan.vocab_size, max_model_len=self.max_model_len,
                                       dtype=self.dtype, device=self.device, workspace=self.workspace, err=self.err)
        # Where a sampler leaves its ids for a step that runs before the host has seen them: one id
        # per request of the batch, and the step's error word behind them.
        self.sampled_tokens = torch.zeros(self.max_num_seqs + 1, dtype=torch.int32, device=self.device)
        self.assembler.sampled = self.sampled_tokens[: self.max_num_seqs]
        self.poison_freed_pages = bool(poison_freed_pages)
        if self.poison_freed_pages:
            self.cache.log_freed(True)
        self.pages_poisoned = 0
        self.steps_run = 0
        self.last_launches = 0      # kernels of ours launched by the last step
        self.last_used_graph = False
        self._graphs: Dict[Tuple[int, Tuple[int, ...]], _DecodeGraph] = {}
        self._graph_workspace: Optional[Workspace] = None
        self._graph_pool = None

    @classmethod
    def random(cls, config_dict: Mapping[str, Any], seed: int, dtype="bfloat16", **kw) -> "ModelRunner":
        """A runner over a model with random weights drawn on the device (nothing is written)."""
        from ..weights.random_init import RandomWeightStore
        device = kw.get("device", "cuda:0")
        entry, cfg = config_from_dict(config_dict)
        plan = entry.plan_of(cfg)
        model = DecoderModel(plan, _dtype_of(dtype), device)
        torch.cuda.set_device(torch.device(device))
        model.load(RandomWeightStore(model_weight_specs(plan), seed, plan.init_std, plan.norm_init_std))
        return cls(None, dtype, model=model, **kw)

    # ---- caches --------------------------------------------------------------------------------------
    def _build_caches(self, num_blocks: Optional[int], kv_fraction: float) -> None:
        """Page pools and page tensors from what the mixers ask for.  Runs that own pages are
        grouped by (window, page size): a group has one pool and one block table per request;
        every run of a group holds its own page tensors, addressed by the group's page ids.
        ``num_blocks`` counts pages of the engine's ``block_size``; a group with another page size
        gets as many pages as hold the same number of tokens."""
        needs = self.model.cache_needs()
        runs = self.plan.runs
        keys: List[Tuple[Optional[int], int]] = []
        run_group: Dict[int, int] = {}
        for pos, (run, need) in enumerate(zip(runs, needs)):
            if need is None or run.cache_from is not None:
                continue
            key = (need.window, int(need.page_size or self.block_size))
            if key[1] <= 0:
                raise StepError(f"layer run {pos} asks for a page size of {key[1]}")
            if key not in keys:
                keys.append(key)
            run_group[pos] = keys.index(key)
        token_bytes = [0] * max(len(keys), 1)     # bytes one cached token takes in each group
        for pos, g in run_group.items():
            token_bytes[g] += needs[pos].bytes_per_token(self.dtype)
        if num_blocks is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(free * kv_fraction)
            total = sum(token_bytes) * self.block_size or 1
            num_blocks = max(budget // total, 1)
            # no group needs more pages than every request at full length
            num_blocks = min(num_blocks, self.max_num_seqs * ((self.max_model_len + self.block_size - 1) // self.block_size))
        self.num_blocks = int(num_blocks)
        self.kv_bytes_per_token = sum(token_bytes)
        tokens = self.num_blocks * self.block_size
        groups = [CacheGroup(ps, max(tokens // ps, 1), w) for w, ps in keys]
        if not groups:
            # no mixer caches anything: one group of bookkeeping alone (no device memory) that never runs
            # out, so that requests still have lengths and slots
            groups = [CacheGroup(self.block_size, self.max_num_seqs * ((self.max_model_len + self.block_size - 1) // self.block_size), None)]
        self.cache = CacheManager(groups, self.max_num_seqs)
        self.layer_caches: List[Optional[LayerCache]] = [None] * len(runs)
        for pos, g in run_group.items():
            grp = groups[g]
            pages = {name: torch.zeros(t.page_shape(grp.num_pages, grp.page_size), dtype=t.dtype or self.dtype,
                                       device=self.device)
                     for name, t in needs[pos].tensors}
            self.layer_caches[pos] = LayerCache(pages, g, grp.page_size)
        for pos, run in enumerate(runs):
            if run.cache_from is not None and needs[pos] is not None and self.layer_caches[run.cache_from] is None:
                raise StepError(f"layer run {pos} reads the cache of run {run.cache_from}, which has none")
        # fixed-size per-request state
        self.state = StateSlots(self.max_num_seqs, self.device)
        self.layer_states: List[Optional[Dict[str, torch.Tensor]]] = []
        for pos, need in enumerate(self.model.state_needs()):
            if not need:
                self.layer_states.append(None)
                continue
            self.layer_states.append({name: self.state.add(f"run{pos}.{name}", shape, dt)
                                      for name, (shape, dt) in need.items()})
        self.has_state = any(s is not None for s in self.layer_states)
        # decode steps may be replayed from CUDA graphs when every part takes the step from device tensors
        self._graph_safe = self.model.graph_safe()

    def kv_cache_tokens(self) -> int:
        return self.num_blocks * self.block_size

    def available_kv_tokens(self) -> int:
        return min(self.cache.free_pages(g) * grp.page_size for g, grp in enumerate(self.cache.groups))

    # ---- requests ----------------------------------------------------------------------------------
    def open_request(self) -> int:
        slot = self.cache.open_request()
        self.state.clear_slot(slot)
        return slot

    def close_request(self, slot: int) -> None:
        self.cache.close_request(slot)

    def prepare_slot(self, slot: int) -> None:
        """Clear a slot's per-request state (for callers that open slots through the scheduler)."""
        self.state.clear_slot(slot)

    # ---- the step --------------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepInput], *, allow_graph: bool = False) -> torch.Tensor:
        """Run one batch; returns float32 logits ``[wanted, vocab]`` on the device (a view of a
        reused buffer: copy what must outlive the next step).

        A token id ``-1 - i`` stands for ``sampled_tokens[i]``: the id that a sampler has left on the
        device and the host has not seen yet (see ``ahead_token``)."""
        if tracing.ENABLED:
            counts = [len(e.tokens) for e in entries]
            tracing.push(f"{tracing.step_kind(counts)} step: {sum(counts)} tokens of {len(counts)} requests")
            try:
                return self._step(entries, allow_graph)
            finally:
                tracing.pop()
        return self._step(entries, allow_graph)

    def _poison_freed(self) -> None:
        """Fill the pages that went back to their pools since the last step with NaN (integer tensors:
        their lowest value).  It is queued before this step's kernels, so a page that was taken again
        at once is poisoned first and written afterwards."""
        by_group: Dict[int, List[int]] = {}
        for g, page in self.cache.drain_freed():
            by_group.setdefault(g, []).append(page)
        for g, pages in by_group.items():
            idx = torch.tensor(sorted(set(pages)), dtype=torch.long, device=self.device)
            for lc in self.layer_caches:
                if lc is None or lc.group != g:
                    continue
                for t in lc.tensors.values():
                    t.index_fill_(0, idx, float("nan") if t.is_floating_point() else torch.iinfo(t.dtype).min)
            self.pages_poisoned += int(idx.numel())

    def _step(self, entries: Sequence[StepInput], allow_graph: bool) -> torch.Tensor:
        if self.poison_freed_pages:
            self._poison_freed()
        if allow_graph and self._graph_eligible(entries):
            return self._step_graph(entries)
        before = kernels.launch_count()
        ctx = self.assembler.prepare(entries)
        logits = self.model.forward(ctx, self.layer_caches, self.layer_states)
        self.finish(entries)
        self.last_launches = kernels.launch_count() - before
        self.last_used_graph = False
        return logits

    @staticmethod
    def ahead_token(i: int) -> int:
        """The token id that tells a step to read ``sampled_tokens[i]`` on the device."""
        return -1 - int(i)

    def finish(self, entries: Sequence[StepInput]) -> None:
        for e in entries:
            self.cache.advance(e.slot, self.cache.length(e.slot) + len(e.tokens))
        self.steps_run += 1

    # ---- decode steps from a CUDA graph ---------------------------------------------------------------
    def _graph_eligible(self, entries: Sequence[StepInput]) -> bool:
        if self.dtype != torch.bfloat16 or not self._graph_safe:
            return False
        for e in entries:
            if len(e.tokens) != 1 or len(e.want) != 1:
                return False
        return True

    def _graph_strides(self, entries: Sequence[StepInput]) -> Tuple[int, ...]:
        longest = max(self.cache.length(e.slot) for e in entries) + 1
        out = []
        for grp in self.cache.groups:
            pages = (longest + grp.page_size - 1) // grp.page_size
            s = 64
            while s < pages:
                s *= 2
            out.append(s)
        return tuple(out)

    def _step_graph(self, entries: Sequence[StepInput]) -> torch.Tensor:
        B = len(entries)
        bucket = _bucket(B, self.max_num_seqs)
        strides = self._graph_strides(entries)
        key = (bucket, strides)
        g = self._graphs.get(key)
        if g is None:
            g = self._capture(entries, bucket, strides)
            self._graphs[key] = g
        self.assembler.prepare(entries, pad_entries=bucket, pad_tokens=bucket, pad_rows=bucket, strides=strides,
                               into=g.meta, workspace=self._graph_workspace)
        g.graph.replay()
        self.finish(entries)
        self.last_launches = g.launches
        self.last_used_graph = True
        return g.logits[:B]

    def _capture(self, entries: Sequence[StepInput], bucket: int, strides: Tuple[int, ...]) -> _DecodeGraph:
        if self._graph_workspace is None:
            self._graph_workspace = Workspace(self.device)
            self._graph_pool = torch.cuda.graph_pool_handle()
        ws = self._graph_workspace
        cap = 3 * (bucket + 4) + 3 * (bucket + 5) + bucket + 8 + sum(bucket * s + 4 for s in strides) + 64
        meta = torch.zeros(cap, dtype=torch.int32, device=self.device)
        kw = dict(pad_entries=bucket, pad_tokens=bucket, pad_rows=bucket, strides=strides, workspace=ws)
        saved_state = {name: t.clone() for name, t in self.state.tables.items()} if self.has_state else None
        # size every buffer for the largest bucket first, so that no later capture moves them
        if not getattr(ws, "sized", False):
            ws.frozen = False
            top = _bucket(self.max_num_seqs, self.max_num_seqs)
            wide = []
            for grp in self.cache.groups:
                widest = 64
                while widest * grp.page_size < self.max_model_len:
                    widest *= 2
                wide.append(widest)
            wide = tuple(wide)
            tmp = torch.zeros(3 * (top + 4) + 3 * (top + 5) + top + 8 + sum(top * s + 4 for s in wide) + 64,
                              dtype=torch.int32, device=self.device)
            # every bucket that _bucket can give, once (scratch sizes are not monotonic in the batch
            # size), largest first: the powers of two below the most requests, and that number itself
            sizes = [top]
            b = 1
            while b < top:
                sizes.append(b)
                b *= 2
            for b in sorted(set(sizes), reverse=True):
                big = self.assembler.prepare(entries[:b], pad_entries=b, pad_tokens=b, pad_rows=b, strides=wide,
                                             into=tmp, workspace=ws)
                self.model.forward(big, self.layer_caches, self.layer_states)
            torch.cuda.current_stream().synchronize()
            del tmp
            ws.sized = True
            ws.frozen = True
        ctx = self.assembler.prepare(entries, into=meta, **kw)
        self.model.forward(ctx, self.layer_caches, self.layer_states)   # warm-up on this stream
        torch.cuda.current_stream().synchronize()
        if saved_state is not None:
            # the passes above ran this step's tokens for real: pages take the same values again when the
            # step is replayed, per-request state would not - it goes back to what it was
            for name, t in saved_state.items():
                self.state.tables[name].copy_(t)
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count()
        ctx.scratch.clear()   # what parts decide once per step (and launch kernels for) is decided again, inside the graph
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(ctx, self.layer_caches, self.layer_states)
        launches = kernels.launch_count() - before
        return _DecodeGraph(graph, meta, logits, launches)

    # ---- errors the kernels reported ---------------------------------------------------------------------
    def queue_error_check(self) -> None:
        """Queue the copy of the device error word; ``raise_if_error`` reads it after the caller's
        next synchronisation (so a step costs one synchronisation, not two)."""
        self._err_host.copy_(self.err, non_blocking=True)

    def raise_if_error(self) -> None:
        word = int(self._err_host[0])
        self._err_host[0] = 0
        self.raise_on(word)

    def raise_on(self, word: int) -> None:
        """Raise for an error word that was read from the device (0: nothing happened)."""
        if word:
            self.err.zero_()
            raise StepError("a kernel reported: " + kernels.describe_error(word))

    def recover(self) -> None:
        """After a failed step: wait for what is queued on the device, clear the error word and
        every scratch buffer (kernels keep counters there that must be zero between launches).
        Pages, weights and captured graphs stay as they are."""
        torch.cuda.synchronize(self.device)
        self.err.zero_()
        self._err_host[0] = 0
        self.workspace.clear()
        if self._graph_workspace is not None:
            self._graph_workspace.clear()
        self.sampled_tokens.zero_()
        torch.cuda.synchronize(self.device)

    def check_errors(self) -> None:
        """Synchronises and raises if any kernel has set the device error word since the last check."""
        self._err_host.copy_(self.err, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.raise_if_error()
