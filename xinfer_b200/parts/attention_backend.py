"""Chooses the attention kernels for a step.

bfloat16 with a head size in steps of 16 up to 256 runs on the tensor-core kernels: portions of
more than ``DEC_MAX`` tokens on the prefill kernel, the tokens of smaller portions on the
split-range decode kernel (both read the same metadata and skip what is not theirs, so one batch
may hold both).  Everything else (float32, other head sizes) runs on the plain kernel.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels

# portions up to this many tokens are treated token by token by the decode kernel
DEC_MAX = 4
# CTAs of the decode kernel that are resident at once (three per SM of a 148-SM part): key ranges
# are cut so that one wave holds them all
DECODE_RESIDENT_CTAS = 444
# what starting a CTA of the decode kernel costs, in key positions of work
DECODE_CTA_OVERHEAD = 96
# the tcgen05 decode kernel: two CTAs per SM; the tiles of all (token, head) pairs are shared out
# evenly among them, but no CTA gets less than this many keys (a CTA's start-up and the merge of a
# shared pair cost about as much as reading 256 keys)
DECODE_TC_CTAS = 296
DECODE_TC_MIN_KEYS = 256
PREFILL_WARPS = 8
# portions of many tokens go to the tcgen05 kernel where it takes the sizes (head size <= 128,
# page size a power of two >= 8), else to the mma.sync kernel
PREFILL_TC = True
# the tokens of small portions go to the tcgen05 decode kernel where it takes the sizes (as above,
# and at most 16 query heads per key/value head), else to the mma.sync kernel
DECODE_TC = True

_enabled = True


def set_tiled(flag: bool) -> None:
    """Switch the tensor-core kernels off (tests compare them with the plain kernel)."""
    global _enabled
    _enabled = bool(flag)


def decode_tc_takes(nh: int, nkv: int, d: int, page_size: int) -> bool:
    return (DECODE_TC and d % 16 == 0 and 16 <= d <= 128 and nh // nkv <= 16 and page_size >= 8
            and page_size & (page_size - 1) == 0)


def prefill_tc_takes(d: int, page_size: int) -> bool:
    return (d % 16 == 0 and 16 <= d <= 128 and page_size >= 8 and page_size & (page_size - 1) == 0
            and kernels.attn_prefill_queries(d, PREFILL_WARPS) == 128)


DECODE_TC_MAX_TOKENS = 8192   # small tokens a plan of the tcgen05 decode kernel takes


def decode_tc_launch(bound: int, tokens: int, kv_heads: int) -> tuple:
    """(ctas, splits_max) of the tcgen05 decode kernel for ``tokens`` tokens whose contexts are at
    most ``bound`` long: as many CTAs as there is work of DECODE_TC_MIN_KEYS keys, up to two per SM."""
    tiles = (max(bound, 1) + 63) // 64
    per = DECODE_TC_MIN_KEYS // 64
    ctas = max(1, min(DECODE_TC_CTAS, (tokens * kv_heads * tiles + per - 1) // per))
    return ctas, kernels.decode_tc_splits_max(ctas, kv_heads, bound, DECODE_TC_MIN_KEYS)


def decode_split(bound: int, pairs: int, resident: int = DECODE_RESIDENT_CTAS, overhead: int = DECODE_CTA_OVERHEAD) -> tuple:
    """Range length (a multiple of 64) and number of ranges for keys up to ``bound`` when
    ``pairs`` (token, key/value head) pairs share the machine.  Each CTA costs its range plus a
    fixed start-up (about ``overhead`` keys' worth); CTAs run in waves of ``resident``.  The cheapest cut wins: few pairs are cut finely so that every SM
    gets work, many pairs coarsely so that little has to be merged and the last wave is full."""
    pairs = max(pairs, 1)
    best = None
    tiles = max((bound + 63) // 64, 1)
    for per in range(1, tiles + 1):                # 64-key tiles per range
        n = (tiles + per - 1) // per
        if n > 1024:
            continue
        if best is not None and per > 1 and (tiles + per - 2) // (per - 1) == n:
            continue                               # same number of ranges as the shorter cut
        waves = (pairs * n + resident - 1) // resident
        cost = waves * (per * 64 + overhead)
        if best is None or cost < best[0]:
            best = (cost, per * 64, n)
    return best[1], best[2]


def _plan(ctx, head_dim: int):
    """Per-step launch figures, computed once and shared by all layers of the step."""
    key = ("attn_plan", head_dim)
    plan = ctx.scratch.get(key)
    if plan is None:
        if ctx.fixed_shapes:
            # a captured step: every token is its own one-token portion; sizes come from the padding
            plan = dict(tiles=0, small=ctx.num_tokens, direct=True, bound=None, prefill_bound=0)
        else:
            counts = np.diff(ctx.h_q_start[: ctx.real_entries + 1])
            small = counts <= DEC_MAX
            per = kernels.attn_prefill_queries(head_dim, PREFILL_WARPS)
            ends = ctx.h_start_pos[: ctx.real_entries] + counts
            plan = dict(tiles=int(((counts[~small] + per - 1) // per).sum()), small=int(counts[small].sum()),
                        direct=bool(small.all()), bound=int(ends[small].max()) if small.any() else 0,
                        prefill_bound=int(ends[~small].max()) if (~small).any() else 0)
        ctx.scratch[key] = plan
    return plan


class _PinnedRing:
    """A few pinned staging buffers used in turn; one is reused only after the copy that read it has
    finished (pinning memory anew for every step would synchronise the device)."""

    def __init__(self, depth: int = 4):
        self.bufs = [None] * depth
        self.events = [None] * depth
        self.i = 0

    def take(self, n: int) -> torch.Tensor:
        self.i = (self.i + 1) % len(self.bufs)
        if self.events[self.i] is not None:
            self.events[self.i].synchronize()
        buf = self.bufs[self.i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 4096), dtype=torch.int32).pin_memory()
            self.bufs[self.i] = buf
        return buf

    def sent(self) -> None:
        ev = torch.cuda.Event()
        ev.record()
        self.events[self.i] = ev


_work_ring = _PinnedRing()


def _prefill_work(ctx, nh: int, nkv: int, window):
    """The step's work list of the tcgen05 prefill kernel for this head layout and window, made once
    per step (natively, on the host) and sent before the step's first kernel; shared by all layers."""
    key = ("attn_prefill_work", nh, nkv, window)
    made = ctx.scratch.get(key)
    if made is None:
        counts = np.diff(ctx.h_q_start[: ctx.real_entries + 1])
        host, ctas = kernels.attn_prefill_work(counts, ctx.h_start_pos[: ctx.real_entries], DEC_MAX, window, nh, nkv,
                                               host_buffer=_work_ring.take)
        made = (host.to(ctx.positions.device, non_blocking=True), ctas, host)
        _work_ring.sent()
        ctx.scratch[key] = made
    return made


def _decode_plan(ctx, nh: int, nkv: int, d: int, page_size: int, window, stride: int, early: bool):
    """The step's plan of the tcgen05 decode kernel for this head layout and window: made once per
    step and shared by all layers.  ``early``: the call comes before the step's first kernel.
    Returns None when the kernel does not take the step, else (plan, ctas, splits_max, overlap)."""
    key = ("attn_decode_plan", nh, nkv, d, page_size, window)
    if key in ctx.scratch:
        return ctx.scratch[key]
    made = None
    plan = _plan(ctx, d)
    small = plan["small"]
    if small and decode_tc_takes(nh, nkv, d, page_size) and small <= DECODE_TC_MAX_TOKENS:
        bound = plan["bound"] if plan["bound"] is not None else stride * page_size
        ctas, splits_max = decode_tc_launch(bound, small, nkv)
        buf = ctx.workspace.get(f"attn.plan.{nkv}.{window or 0}", (kernels.attn_decode_plan_size(small, ctas, nkv),), torch.int32)
        if kernels.attn_decode_plan(buf, ctx.positions, ctx.req_of_token, ctx.q_start, ctx.num_entries, window, DEC_MAX,
                                    plan["direct"], small, DECODE_TC_MIN_KEYS, ctas, nkv, ctx.err):
            # a plan made in the middle of the step is read only after the kernel before has completed
            made = (buf, ctas, splits_max, bool(early))
    ctx.scratch[key] = made
    return made


def prepare_step(ctx, dtype, nh: int, nkv: int, d: int, page_size: int, window, stride: int) -> None:
    """Called before the step's first kernel for every attention layer (``stride``: the width of
    its block table): plans the decode kernel."""
    if _enabled and kernels.attn_tiled_supported(dtype, d):
        _decode_plan(ctx, nh, nkv, d, page_size, window, stride, early=True)
        if _plan(ctx, d)["tiles"] and PREFILL_TC and prefill_tc_takes(d, page_size):
            _prefill_work(ctx, nh, nkv, window)


def attend(out, q, cache, ctx, table, stride, window, scale) -> None:
    T, nh, d = q.shape
    k_pages, v_pages = cache["k"], cache["v"]
    if not (_enabled and kernels.attn_tiled_supported(q.dtype, d)):
        kernels.attention_plain(out, q, k_pages, v_pages, ctx.positions, ctx.req_of_token, table, stride,
                                window, scale, ctx.err)
        return
    plan = _plan(ctx, d)
    took = False
    if plan["tiles"] and PREFILL_TC and prefill_tc_takes(d, cache.page_size):
        work, ctas, _ = _prefill_work(ctx, nh, k_pages.shape[1], window)
        took = kernels.attn_prefill_tc(out, q, k_pages, v_pages, ctx.q_start, ctx.start_pos, table, stride, window, scale,
                                       work, ctas, ctx.err)
    if plan["tiles"] and not took:
        kernels.attn_prefill_bf16(out, q, k_pages, v_pages, ctx.q_start, ctx.start_pos, ctx.num_entries, table, stride,
                                  window, scale, DEC_MAX, plan["tiles"], plan["prefill_bound"], ctx.err, warps=PREFILL_WARPS)
    if plan["small"]:
        nkv = k_pages.shape[1]
        bound = plan["bound"] if plan["bound"] is not None else stride * cache.page_size
        small = plan["small"]
        part_o = part_ml = tickets = None

        def scratch(splits):
            nonlocal part_o, part_ml, tickets
            if splits > 1:
                part_o = ctx.workspace.get("attn.part_o", (small * nh * splits * d,), torch.float32)
                part_ml = ctx.workspace.get("attn.part_ml", (small * nh * splits * 2,), torch.float32)
                # zero-filled when made, left zero by the kernels; sized for either kernel
                tickets = ctx.workspace.get("attn.tickets", (small * nkv * ((nh // nkv + 15) // 16),), torch.int32)

        step = (q, k_pages, v_pages, ctx.positions, ctx.req_of_token, ctx.q_start, ctx.num_entries, table, stride,
                window, scale, DEC_MAX, plan["direct"])
        took = False
        planned = _decode_plan(ctx, nh, nkv, d, cache.page_size, window, stride, early=False)
        if planned is not None:
            buf, ctas, splits_max, overlap = planned
            scratch(splits_max)
            took = kernels.attn_decode_tc(out, part_o, part_ml, q, k_pages, v_pages, buf, table, stride, scale, DEC_MAX,
                                          splits_max, small, ctas, ctx.err, tickets, overlap)
        if not took:
            split, num_splits = decode_split(bound, small * nkv * ((nh // nkv + 15) // 16))
            scratch(num_splits)
            kernels.attn_decode_bf16(out, part_o, part_ml, *step, split, num_splits, small, ctx.err, tickets)
