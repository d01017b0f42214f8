"""SiLU-gated feed-forward: ``down( silu(gate(x)) * up(x) )`` with gate and up concatenated into
one projection at load (src/models/layers/mlp.rs:447-466, forward :613-697), no biases."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import FeedForwardSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, register_feed_forward
from . import gemm_backend
from .linear import linear


class SwiGLU(FeedForward):
    kind = "swiglu"
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.activation != "silu":
            raise ValueError(f"the gated feed-forward supports 'silu', not '{spec.activation}'")
        self.w_gate_up = self.w_down = None

    @classmethod
    def weight_specs(cls, spec: FeedForwardSpec, prefix: str) -> List[WeightSpec]:
        p = prefix
        return [
            WeightSpec(p + "gate_proj.weight", (spec.intermediate, spec.hidden)),
            WeightSpec(p + "up_proj.weight", (spec.intermediate, spec.hidden)),
            WeightSpec(p + "down_proj.weight", (spec.hidden, spec.intermediate)),
        ]

    def load(self, store) -> None:
        p = self.prefix
        g = store.get(p + "gate_proj.weight", self.device, self.dtype, operand=True)
        u = store.get(p + "up_proj.weight", self.device, self.dtype, operand=True)
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        del g, u
        self.w_down = store.get(p + "down_proj.weight", self.device, self.dtype, operand=True)

    def forward(self, x, ctx: StepContext):
        s = self.spec
        T = x.shape[0]
        ws = ctx.workspace
        act = ws.get("ffn.act", (T, s.intermediate), self.dtype)
        if not gemm_backend.try_fused_gate(act, x, self.w_gate_up, ctx.err):
            gu = ws.get("ffn.gate_up", (T, 2 * s.intermediate), self.dtype)
            linear(gu, x, self.w_gate_up, ctx.err)
            kernels.swiglu(act, gu)
        out = ws.get("ffn.out", (T, s.hidden), self.dtype)
        linear(out, act, self.w_down, ctx.err)
        return out


register_feed_forward("swiglu", SwiGLU)
