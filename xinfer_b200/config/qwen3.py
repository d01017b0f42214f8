"""Typed configuration of the Qwen3 dense decoder, read from the keys of its own config.json.

Keys and defaults follow what the reference reads for this architecture
(src/utils/config.rs:277-330 for the struct; src/models/layers/attention.rs:446 for the
``head_dim`` default; src/models/layers/rotary_emb.rs:49 for the ``rope_theta`` default;
src/models/qwen3.rs:200-209, 267-287 for tied/untied heads).  Every size used anywhere in the
engine comes from here; nothing is hard-coded.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .plan import (AttentionSpec, FeedForwardSpec, LayerRun, ModelPlan, NormSpec, RopeSpec,
                   pre_norm_block)


_REQUIRED = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "max_position_embeddings",
)


def _as_int(raw: Mapping[str, Any], key: str) -> int:
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config key '{key}' must be an integer, got {v!r}")
    if v <= 0:
        raise ConfigError(f"config key '{key}' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    # The reference hands ``sliding_window`` to every layer's attention when the key holds a
    # number (src/models/qwen3.rs:37-48); ``use_sliding_window`` / ``max_window_layers`` are parsed
    # and never read (src/utils/config.rs:299-301).  The same rule is kept here.
    sliding_window: Optional[int] = None
    hidden_act: str = "silu"
    attention_bias: bool = False
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)

    ARCHITECTURE = "Qwen3ForCausalLM"

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in raw or raw[k] is None]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        ints = {k: _as_int(raw, k) for k in _REQUIRED if k != "rms_norm_eps"}
        eps = raw["rms_norm_eps"]
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not (eps > 0):
            raise ConfigError(f"config key 'rms_norm_eps' must be a positive number, got {eps!r}")
        nh, nkv, hidden = ints["num_attention_heads"], ints["num_key_value_heads"], ints["hidden_size"]
        if raw.get("head_dim") is not None:
            head_dim = _as_int(raw, "head_dim")
        else:
            if hidden % nh:
                raise ConfigError(
                    f"'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {nh}")
            head_dim = hidden // nh
        if nh % nkv:
            raise ConfigError(f"num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for rotary position encoding")
        act = raw.get("hidden_act", raw.get("hidden_activation", "silu"))
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported (the gated feed-forward uses 'silu')")
        if raw.get("attention_bias") or raw.get("qkv_bias"):
            raise ConfigError("attention_bias=true is not supported by this architecture entry")
        scaling = raw.get("rope_scaling", raw.get("rope_parameters"))
        if scaling:
            kind = scaling.get("rope_type", scaling.get("type", "default")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise ConfigError(f"rope_scaling '{kind}' is not supported (only the default rotary tables)")
        window = raw.get("sliding_window")
        if window is not None:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"config key 'sliding_window' must be a positive integer or null, got {window!r}")
        theta = raw.get("rope_theta")
        if theta is None and isinstance(scaling, dict):
            theta = scaling.get("rope_theta")
        if theta is None:
            theta = 10000.0
        if isinstance(theta, bool) or not isinstance(theta, (int, float)) or not (theta > 0):
            raise ConfigError(f"config key 'rope_theta' must be a positive number, got {theta!r}")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config key 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
        archs = raw.get("architectures") or [cls.ARCHITECTURE]
        return cls(
            vocab_size=ints["vocab_size"], hidden_size=hidden,
            intermediate_size=ints["intermediate_size"],
            num_hidden_layers=ints["num_hidden_layers"], num_attention_heads=nh,
            num_key_value_heads=nkv, head_dim=head_dim, rms_norm_eps=float(eps),
            rope_theta=float(theta), max_position_embeddings=ints["max_position_embeddings"],
            tie_word_embeddings=bool(raw.get("tie_word_embeddings") or False),
            sliding_window=window, hidden_act=act, attention_bias=False, eos_token_id=eos_ids,
            bos_token_id=raw.get("bos_token_id"), architectures=tuple(archs),
        )

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        eos = list(self.eos_token_id)
        d["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        d["model_type"] = "qwen3"
        d["use_sliding_window"] = self.sliding_window is not None
        return d

    # ---- the arrangement of parts ---------------------------------------------------------
    def plan(self) -> ModelPlan:
        """Every layer: RMSNorm -> grouped-query attention with per-head q/k RMSNorm and NeoX
        rotary encoding -> RMSNorm -> SiLU-gated feed-forward (src/models/qwen3.rs:108-134)."""
        rope = RopeSpec(kind="rope", head_dim=self.head_dim, rotary_dim=self.head_dim,
                        theta=self.rope_theta, max_positions=self.max_position_embeddings,
                        layout="neox")
        blocks = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            blocks.append(pre_norm_block(
                prefix=p,
                norm_in=NormSpec(kind="rmsnorm", dim=self.hidden_size, eps=self.rms_norm_eps),
                mixer=AttentionSpec(
                    kind="attention", hidden=self.hidden_size, num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                    scale=1.0 / math.sqrt(self.head_dim), qk_norm=True,
                    qk_norm_eps=self.rms_norm_eps, rope=rope, window=self.sliding_window),
                norm_post=NormSpec(kind="rmsnorm", dim=self.hidden_size, eps=self.rms_norm_eps),
                feed_forward=FeedForwardSpec(kind="swiglu", hidden=self.hidden_size,
                                             intermediate=self.intermediate_size,
                                             activation=self.hidden_act),
            ))
        plan = ModelPlan(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab_size, hidden=self.hidden_size,
            embed_name="model.embed_tokens.weight", blocks=tuple(blocks),
            runs=tuple(LayerRun(block=i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec(kind="rmsnorm", dim=self.hidden_size, eps=self.rms_norm_eps),
            final_norm_name="model.norm.",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            max_positions=self.max_position_embeddings, eos_token_ids=self.eos_token_id,
        )
        plan.validate()
        return plan
