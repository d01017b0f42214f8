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
PREFILL_WARPS = 8
# portions of many tokens go to the tcgen05 kernel where it takes the sizes (head size <= 128,
# page size a power of two >= 8), else to the mma.sync kernel
PREFILL_TC = True

_enabled = True


def set_tiled(flag: bool) -> None:
    """Switch the tensor-core kernels off (tests compare them with the plain kernel)."""
    global _enabled
    _enabled = bool(flag)


def decode_split(bound: int, pairs: int) -> tuple:
    """Range length (a multiple of 64) and number of ranges for keys up to ``bound`` when
    ``pairs`` (token, key/value head) pairs share the machine.  Each CTA costs its range plus a
    fixed start-up (about ``DECODE_CTA_OVERHEAD`` keys' worth); CTAs run in waves of
    ``DECODE_RESIDENT_CTAS``.  The cheapest cut wins: few pairs are cut finely so that every SM
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
        waves = (pairs * n + DECODE_RESIDENT_CTAS - 1) // DECODE_RESIDENT_CTAS
        cost = waves * (per * 64 + DECODE_CTA_OVERHEAD)
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


def attend(out, q, cache, ctx, table, stride, window, scale) -> None:
    T, nh, d = q.shape
    if not (_enabled and kernels.attn_tiled_supported(q.dtype, d)):
        kernels.attention_plain(out, q, cache.k, cache.v, ctx.positions, ctx.req_of_token, table, stride,
                                window, scale, ctx.err)
        return
    plan = _plan(ctx, d)
    took = False
    if plan["tiles"] and PREFILL_TC and kernels.attn_prefill_queries(d, PREFILL_WARPS) == 128:
        took = kernels.attn_prefill_tc(out, q, cache.k, cache.v, ctx.q_start, ctx.start_pos, ctx.num_entries, table, stride,
                                       window, scale, DEC_MAX, plan["tiles"], ctx.err)
    if plan["tiles"] and not took:
        kernels.attn_prefill_bf16(out, q, cache.k, cache.v, ctx.q_start, ctx.start_pos, ctx.num_entries, table, stride,
                                  window, scale, DEC_MAX, plan["tiles"], plan["prefill_bound"], ctx.err, warps=PREFILL_WARPS)
    if plan["small"]:
        nkv = cache.k.shape[1]
        bound = plan["bound"] if plan["bound"] is not None else stride * cache.page_size
        pairs = plan["small"] * nkv * ((nh // nkv + 15) // 16)
        split, num_splits = decode_split(bound, pairs)
        part_o = part_ml = tickets = None
        if num_splits > 1:
            part_o = ctx.workspace.get("attn.part_o", (plan["small"] * nh * num_splits * d,), torch.float32)
            part_ml = ctx.workspace.get("attn.part_ml", (plan["small"] * nh * num_splits * 2,), torch.float32)
            tickets = ctx.workspace.get("attn.tickets", (pairs,), torch.int32)   # zero-filled when made, left zero
        kernels.attn_decode_bf16(out, part_o, part_ml, q, cache.k, cache.v, ctx.positions, ctx.req_of_token, ctx.q_start,
                                 ctx.num_entries, table, stride, window, scale, DEC_MAX, plan["direct"], split, num_splits,
                                 plan["small"], ctx.err, tickets)
