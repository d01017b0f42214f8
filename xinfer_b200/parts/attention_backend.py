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

_enabled = True


def set_tiled(flag: bool) -> None:
    """Switch the tensor-core kernels off (tests compare them with the plain kernel)."""
    global _enabled
    _enabled = bool(flag)


def _plan(ctx):
    """Per-step launch figures, computed once and shared by all layers of the step."""
    plan = ctx.scratch.get("attn_plan")
    if plan is None:
        if ctx.fixed_shapes:
            # a captured step: every token is its own one-token portion; sizes come from the padding
            plan = dict(tiles=0, small=ctx.num_tokens, direct=True, bound=None)
        else:
            counts = np.diff(ctx.h_q_start[: ctx.real_entries + 1])
            small = counts <= DEC_MAX
            plan = dict(tiles=int(((counts[~small] + 63) // 64).sum()), small=int(counts[small].sum()),
                        direct=bool(small.all()), bound=int(ctx.max_context))
        ctx.scratch["attn_plan"] = plan
    return plan


def attend(out, q, cache, ctx, table, stride, window, scale) -> None:
    T, nh, d = q.shape
    if not (_enabled and kernels.attn_tiled_supported(q.dtype, d)):
        kernels.attention_plain(out, q, cache.k, cache.v, ctx.positions, ctx.req_of_token, table, stride,
                                window, scale, ctx.err)
        return
    plan = _plan(ctx)
    if plan["tiles"]:
        kernels.attn_prefill_bf16(out, q, cache.k, cache.v, ctx.q_start, ctx.start_pos, ctx.num_entries, table, stride,
                                  window, scale, DEC_MAX, plan["tiles"], ctx.err)
    if plan["small"]:
        bound = plan["bound"] if plan["bound"] is not None else stride * cache.page_size
        split = kernels.attn_decode_split()
        num_splits = max((bound + split - 1) // split, 1)
        part_o = part_ml = None
        if num_splits > 1:
            part_o = ctx.workspace.get("attn.part_o", (plan["small"] * nh * num_splits * d,), torch.float32)
            part_ml = ctx.workspace.get("attn.part_ml", (plan["small"] * nh * num_splits * 2,), torch.float32)
        kernels.attn_decode_bf16(out, part_o, part_ml, q, cache.k, cache.v, ctx.positions, ctx.req_of_token, ctx.q_start,
                                 ctx.num_entries, table, stride, window, scale, DEC_MAX, plan["direct"], num_splits,
                                 plan["small"], ctx.err)
