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
# the tcgen05 decode kernel: two CTAs per SM; times in microseconds measured on a B200 at head size 128
DECODE_TC_SMS = 148
DECODE_TC_CTA_LATENCY = 7.5      # a CTA's start-up and merge
DECODE_TC_TILE_ALONE = 0.9       # one 64-key tile of a CTA that has its SM to itself (latency-bound)
DECODE_TC_TILE_SHARED = 1.16     # the same when two CTAs share the SM's path to memory
DECODE_TC_MERGE_LATENCY = 0.1    # per range the last CTA merges
DECODE_TC_TILE_HBM = 0.005       # one tile's keys and values at the memory's full rate
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


def decode_split_tc(bound: int, pairs: int, head_dim: int = 128, page_size: int = 16) -> tuple:
    """Longest range (a multiple of 64) and number of ranges for the tcgen05 decode kernel.  The
    time of a cut is that of the busiest SM - its CTAs run two at a time, each start-up, tiles and
    merge - or what the memory's rate allows for all tiles, whichever is larger; the cheapest cut
    wins.  A range stays within the 1,000 block-table entries that a CTA stages in shared memory."""
    pairs = max(pairs, 1)
    tiles = max((bound + 63) // 64, 1)
    width = max(head_dim, 64) / 128.0
    shared = max(DECODE_TC_TILE_ALONE, DECODE_TC_TILE_SHARED * width)
    floor = pairs * tiles * DECODE_TC_TILE_HBM * width
    best = None
    last_n = None
    for per in range(1, min(tiles, max(1000 * page_size // 64, 1)) + 1):
        n = (tiles + per - 1) // per
        if n > 1024 or n == last_n:
            continue
        last_n = n
        on_sm = (pairs * n + DECODE_TC_SMS - 1) // DECODE_TC_SMS
        rounds = (on_sm + 1) // 2
        tile = shared if on_sm >= 2 else DECODE_TC_TILE_ALONE
        cost = max(rounds * (DECODE_TC_CTA_LATENCY + tile * per + DECODE_TC_MERGE_LATENCY * n), floor)
        if best is None or cost <= best[0] + 1e-9:   # on a tie the longer ranges: less to merge
            best = (cost, per * 64, n)
    return best[1], best[2]


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
        tc = decode_tc_takes(nh, nkv, d, cache.page_size)
        if tc:
            pairs = plan["small"] * nkv
            split, num_splits = decode_split_tc(bound, pairs, d, cache.page_size)
        else:
            pairs = plan["small"] * nkv * ((nh // nkv + 15) // 16)
            split, num_splits = decode_split(bound, pairs)
        part_o = part_ml = tickets = None
        if num_splits > 1:
            part_o = ctx.workspace.get("attn.part_o", (plan["small"] * nh * num_splits * d,), torch.float32)
            part_ml = ctx.workspace.get("attn.part_ml", (plan["small"] * nh * num_splits * 2,), torch.float32)
            # zero-filled when made, left zero by the kernels; sized for either kernel
            tickets = ctx.workspace.get("attn.tickets", (plan["small"] * nkv * ((nh // nkv + 15) // 16),), torch.int32)
        args = (out, part_o, part_ml, q, cache.k, cache.v, ctx.positions, ctx.req_of_token, ctx.q_start,
                ctx.num_entries, table, stride, window, scale, DEC_MAX, plan["direct"], split, num_splits,
                plan["small"], ctx.err, tickets)
        if not (tc and kernels.attn_decode_tc(*args)):
            kernels.attn_decode_bf16(*args)
