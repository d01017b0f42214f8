"""Grouped-query attention over the paged cache.

Order of operations as in the reference (src/models/layers/attention.rs:796-977): one packed
q/k/v projection (:819-828; the three weights are concatenated at load, :376-386), per-head
RMSNorm of q and k before the rotation (:709-748, :869), rotary encoding (:872-879), keys and
values written to their pages and attention over the request's cached positions (:947-958),
then the output projection (:976).  Query head h reads key/value head h // (heads / kv_heads)
(:1040-1047).  A query at position p sees keys j with max(0, p - window + 1) <= j <= p.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import AttentionSpec
from ..weights.loader import WeightSpec
from .base import (LayerCache, Mixer, PagedCacheNeed, StepContext, build_part, register_mixer)
from . import gemm_backend
from .linear import linear


class Attention(Mixer):
    kind = "attention"
    graph_safe = True

    def __init__(self, spec: AttentionSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads do not divide into {spec.num_kv_heads} key/value heads")
        self.position = (build_part("position", spec.rope, prefix, dtype, device)
                         if spec.rope is not None else None)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    @classmethod
    def weight_specs(cls, spec: AttentionSpec, prefix: str) -> List[WeightSpec]:
        p = prefix
        d = spec.head_dim
        out = [
            WeightSpec(p + "q_proj.weight", (spec.num_heads * d, spec.hidden)),
            WeightSpec(p + "k_proj.weight", (spec.num_kv_heads * d, spec.hidden)),
            WeightSpec(p + "v_proj.weight", (spec.num_kv_heads * d, spec.hidden)),
            WeightSpec(p + "o_proj.weight", (spec.hidden, spec.num_heads * d)),
        ]
        if spec.qk_norm:
            out += [WeightSpec(p + "q_norm.weight", (d,), "norm"), WeightSpec(p + "k_norm.weight", (d,), "norm")]
        return out

    def load(self, store) -> None:
        p = self.prefix
        # projection matrices take the engine's dtype whatever the file holds (src/models/layers/linear.rs:133-138)
        parts = [store.get(p + n + ".weight", self.device, self.dtype, operand=True) for n in ("q_proj", "k_proj", "v_proj")]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        del parts
        self.w_o = store.get(p + "o_proj.weight", self.device, self.dtype, operand=True)
        if self.spec.qk_norm:
            self.q_norm = store.get(p + "q_norm.weight", self.device, torch.float32).float().contiguous()
            self.k_norm = store.get(p + "k_norm.weight", self.device, torch.float32).float().contiguous()

    def cache_need(self) -> PagedCacheNeed:
        return PagedCacheNeed.keys_and_values(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def prepare_step(self, ctx: StepContext, cache: LayerCache) -> None:
        from . import attention_backend
        s = self.spec
        attention_backend.prepare_step(ctx, self.dtype, s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, s.window,
                                       ctx.strides[cache.group])

    def forward(self, x, ctx: StepContext, cache: LayerCache, state=None, writes_cache: bool = True):
        s = self.spec
        T = x.shape[0]
        nh, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        ws = ctx.workspace
        rot = self.position.rotary() if self.position is not None else None
        q = ws.get("attn.q", (T, nh, d), self.dtype)
        table, stride = ctx.tables[cache.group], ctx.strides[cache.group]
        head_args = (self.q_norm, self.k_norm, rot.cos if rot else None, rot.sin if rot else None, ctx.positions,
                     ctx.req_of_token, table, stride, nh, nkv, d, rot.rotary_dim if rot else 0,
                     rot.interleaved if rot else False, s.qk_norm_eps, writes_cache, ctx.err)
        k_pages, v_pages = cache["k"], cache["v"]
        fused = (self.position is None or rot is not None) and gemm_backend.try_fused_qkv(
            q, k_pages, v_pages, x, self.w_qkv, *head_args)
        if not fused:
            qkv = ws.get("attn.qkv", (T, (nh + 2 * nkv) * d), self.dtype)
            linear(qkv, x, self.w_qkv, ctx.err)
            if self.position is not None and rot is None:
                q_view = qkv[:, : nh * d].view(T, nh, d)
                k_view = qkv[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
                self.position.apply(q_view, k_view, ctx)
            kernels.qk_norm_rope_write(q, k_pages, v_pages, qkv, *head_args)
        o = ws.get("attn.o", (T, nh, d), self.dtype)
        from . import attention_backend
        attention_backend.attend(o, q, cache, ctx, table, stride, s.window, s.scale)
        out = ws.get("attn.out", (T, s.hidden), self.dtype)
        linear(out, o.view(T, nh * d), self.w_o, ctx.err)
        return out


register_mixer("attention", Attention)
