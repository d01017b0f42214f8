"""The generic decoder: builds any ``ModelPlan`` from registered parts and runs one step of it.

embedding (times the plan's ``embed_scale``, if it has one) -> the plan's layer runs in order ->
final norm on the wanted rows -> output head -> the plan's logit scale and soft cap, if any.
(The reference's forward for this architecture: src/models/qwen3.rs:311-374.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import kernels, tracing
from ..config.plan import ModelPlan
from ..parts import Block, LayerCache, StepContext, build_part, part_class
from ..parts.block import Stream
from ..parts.linear import linear
from ..weights.loader import WeightSpec, WeightStore


def model_weight_specs(plan: ModelPlan) -> List[WeightSpec]:
    """Every tensor the model needs, in file order."""
    specs = [WeightSpec(plan.embed_name, (plan.vocab_size, plan.hidden), "embedding")]
    for b in plan.blocks:
        specs += Block.weight_specs(b)
    specs += part_class("norm", plan.final_norm.kind).weight_specs(plan.final_norm, plan.final_norm_name)
    if plan.head_name is not None:
        specs.append(WeightSpec(plan.head_name, (plan.vocab_size, plan.hidden), "linear"))
    names = [s.name for s in specs]
    if len(set(names)) != len(names):
        dup = sorted({n for n in names if names.count(n) > 1})
        raise ValueError("the plan declares tensors twice: " + ", ".join(dup))
    return specs


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device):
        plan.validate()
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks = [Block(b, dtype, self.device) for b in plan.blocks]
        self.final_norm = build_part("norm", plan.final_norm, plan.final_norm_name, dtype, self.device)
        self.embed = None
        self.head = None

    # ---- weights -------------------------------------------------------------------------------
    def load(self, store: WeightStore) -> None:
        store.check(model_weight_specs(self.plan))
        self.embed = store.get(self.plan.embed_name, self.device, self.dtype, operand=True)
        for b in self.blocks:
            b.load(store)
        self.final_norm.load(store)
        self.head = self.embed if self.plan.head_name is None else store.get(
            self.plan.head_name, self.device, self.dtype, operand=True)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        visit(self)
        visit(self.final_norm)
        for b in self.blocks:
            for part in b.all_parts():
                visit(part)
        return total

    def graph_safe(self) -> bool:
        """Every part takes what it needs of a step from device tensors: decode steps can be replayed from CUDA graphs."""
        return self.final_norm.graph_safe and all(p.graph_safe for b in self.blocks for p in b.all_parts())

    # ---- what the runs need from the cache ---------------------------------------------------------
    def cache_needs(self):
        """Per layer run: the mixer's paged-cache need (None if it has none or reads another run's)."""
        out = []
        for run in self.plan.runs:
            mixer = self.blocks[run.block].mixer
            out.append(mixer.cache_need() if mixer is not None else None)
        return out

    def state_needs(self):
        mixers = [self.blocks[run.block].mixer for run in self.plan.runs]
        return [m.state_need() if m is not None else None for m in mixers]

    # ---- one step ------------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: List[Optional[LayerCache]],
                states: List[Optional[Dict[str, torch.Tensor]]]) -> torch.Tensor:
        """Runs the step's tokens through the layer runs and returns float32 logits
        ``[num_logit_rows, vocab]`` for ``ctx.logit_rows``."""
        T, H, V = ctx.num_tokens, self.plan.hidden, self.plan.vocab_size
        ws = ctx.workspace
        x = ws.get("model.x", (T, H), self.dtype)
        # what mixers decide once per step from its metadata, before the step's first kernel
        for pos, run in enumerate(self.plan.runs):
            mixer = self.blocks[run.block].mixer
            if mixer is not None:
                mixer.prepare_step(ctx, caches[pos if run.cache_from is None else run.cache_from])
        trace = tracing.ENABLED
        if trace:
            tracing.push("embedding")
        kernels.embedding(x, self.embed, ctx.token_ids, ctx.err, ctx.sampled, scale=self.plan.embed_scale)
        if trace:
            tracing.pop()
        stream = Stream(x)
        for pos, run in enumerate(self.plan.runs):
            src = pos if run.cache_from is None else run.cache_from
            stream = self.blocks[run.block].forward(stream, ctx, caches[src], states[pos],
                                                    writes_cache=run.cache_from is None)
        R = ctx.num_logit_rows
        logits = ws.get("model.logits", (max(R, 1), V), torch.float32)[:R]
        if R == 0:
            return logits      # nothing reads the stream again: its waiting additions are void
        if trace:
            tracing.push("head")
        y = ws.get("model.final", (R, H), self.dtype)
        self.final_norm.forward(y, stream.x, ctx, branch=stream.settle(keep_last=True), rows=ctx.logit_rows)
        linear(logits, y, self.head, ctx.err)
        if self.plan.logit_scale is not None or self.plan.logit_softcap is not None:
            kernels.logits_post(logits, self.plan.logit_scale, self.plan.logit_softcap)
        if trace:
            tracing.pop()
        return logits
