"""The arrangement of parts in one layer: a pre-norm residual block
``x + mixer(norm_in(x))`` then ``x + feed_forward(norm_post(x))`` (src/models/qwen3.rs:108-134).

The residual sum is fused with the norm that follows it: a block receives the residual stream and
the previous block's not-yet-added branch, and hands back the same pair, so each sum is formed
once, in float32, inside the norm kernel that needs it."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.plan import BlockSpec
from ..weights.loader import WeightSpec
from .base import LayerCache, StepContext, build_part, part_class


class Block:
    def __init__(self, spec: BlockSpec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        p = spec.prefix
        self.norm_in = build_part("norm", spec.norm_in, p + spec.norm_in_name, dtype, device)
        self.mixer = build_part("mixer", spec.mixer, p + spec.mixer_name, dtype, device)
        self.norm_post = build_part("norm", spec.norm_post, p + spec.norm_post_name, dtype, device)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, p + spec.feed_forward_name, dtype, device)

    @staticmethod
    def weight_specs(spec: BlockSpec) -> List[WeightSpec]:
        p = spec.prefix
        return (part_class("norm", spec.norm_in.kind).weight_specs(spec.norm_in, p + spec.norm_in_name)
                + part_class("mixer", spec.mixer.kind).weight_specs(spec.mixer, p + spec.mixer_name)
                + part_class("norm", spec.norm_post.kind).weight_specs(spec.norm_post, p + spec.norm_post_name)
                + part_class("feed_forward", spec.feed_forward.kind).weight_specs(spec.feed_forward, p + spec.feed_forward_name))

    def load(self, store) -> None:
        for part in (self.norm_in, self.mixer, self.norm_post, self.feed_forward):
            part.load(store)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[LayerCache], state, writes_cache: bool):
        """``x``: residual stream; ``pending``: a branch output still to be added to it (or None).
        Returns the new (x, pending)."""
        T, H = x.shape
        h = ctx.workspace.get("block.normed", (T, H), self.dtype)
        if pending is None:
            self.norm_in.forward(h, x, ctx)
        else:
            self.norm_in.forward(h, x, ctx, branch=pending, sum_out=x)
        a = self.mixer.forward(h, ctx, cache, state, writes_cache)
        self.norm_post.forward(h, x, ctx, branch=a, sum_out=x)
        f = self.feed_forward.forward(h, ctx)
        return x, f
