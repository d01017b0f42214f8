"""The generic decoder: builds any ``ModelPlan`` from registered parts and runs one step of it.

embedding -> the plan's layer runs in order -> final norm on the wanted rows -> output head.
(The reference's forward for this architecture: src/models/qwen3.rs:311-374.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..config.plan import ModelPlan
from ..parts import Block, LayerCache, StepContext, build_part, part_class
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
        self.embed = store.get(self.plan.embed_name, self.device, self.dtype)
        for b in self.blocks:
            b.load(store)
        self.final_norm.load(store)
        self.head = self.embed if self.plan.head_name is None else store.get(self.plan.head_name, self.device, self.dtype)

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
            for part in (b.norm_in, b.mixer, b.norm_post, b.feed_forward):
                visit(part)
        return total

    # ---- what the runs need from the cache ---------------------------------------------------------
    def cache_needs(self):
        """Per layer run: the mixer's paged-cache need (None if it has none or reads another run's)."""
        out = []
        for run in self.plan.runs:
            need = self.blocks[run.block].mixer.cache_need()
            out.append(need)
        return out

    def state_needs(self):
        return [self.blocks[run.block].mixer.state_need() for run in self.plan.runs]

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
            src = pos if run.cache_from is None else run.cache_from
            self.blocks[run.block].mixer.prepare_step(ctx, caches[src])
        kernels.embedding(x, self.embed, ctx.token_ids, ctx.err, ctx.sampled)
        pending = None
        for pos, run in enumerate(self.plan.runs):
            src = pos if run.cache_from is None else run.cache_from
            x, pending = self.blocks[run.block].forward(
                x, pending, ctx, caches[src], states[pos], writes_cache=run.cache_from is None)
        R = ctx.num_logit_rows
        logits = ws.get("model.logits", (max(R, 1), V), torch.float32)[:R]
        if R == 0:
            return logits
        y = ws.get("model.final", (R, H), self.dtype)
        self.final_norm.forward(y, x, ctx, branch=pending, rows=ctx.logit_rows)
        linear(logits, y, self.head, ctx.err)
        return logits
