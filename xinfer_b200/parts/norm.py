"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * (offset + w)``, statistics and weight product in
float32 (src/models/layers/others.rs:22-46, 65-85), with the fused form that first adds a branch
to the residual stream and returns both the sum and its norm (others.rs:48-62, 87-125)."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import NormSpec
from ..weights.loader import WeightSpec
from .base import Norm, register_norm


class RMSNorm(Norm):
    kind = "rmsnorm"
    graph_safe = True

    def __init__(self, spec: NormSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.weight = None

    @classmethod
    def weight_specs(cls, spec: NormSpec, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(prefix + "weight", (spec.dim,), "norm")]

    def load(self, store) -> None:
        # norm weights are held in float32 whatever the activations are (src/models/qwen3.rs:83)
        self.weight = store.get(self.prefix + "weight", self.device, torch.float32).float().contiguous()

    def forward(self, out, x, ctx, branch=None, sum_out=None, rows=None):
        kernels.rmsnorm(out, x, self.weight, self.spec.eps, ctx.err, branch=branch, sum_out=sum_out,
                        rows=rows, weight_offset=self.spec.weight_offset)
        return out


register_norm("rmsnorm", RMSNorm)
