"""Typed descriptions of a decoder: what each layer is made of and in which order layers run.

A model is described as data before anything is built:

* a *part spec* per part (mixer, feed-forward, norm, position encoding) carrying every size and
  constant the part needs, so no part ever looks at a model configuration;
* a ``BlockSpec`` per set of weights: which mixer, which feed-forward, which norms;
* a ``LayerRun`` list: the order in which blocks execute.  A block may be named twice (its
  weights are reused, each run keeps a cache of its own), and a run may read the cache that an
  earlier run wrote instead of writing one (``cache_from``).

The reference wires one struct per architecture by hand (src/models/qwen3.rs:20-135 for the
layer, :137-290 for the stack); here the same information is a ``ModelPlan`` that a generic
decoder builds from.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Base of every part spec. ``kind`` selects the implementation in the part registry."""

    kind: str

    def params(self) -> Dict[str, Any]:
        d = dict(self.__dict__)
        d.pop("kind")
        return d


@dataclass(frozen=True)
class RopeSpec(PartSpec):
    """Rotary position encoding over the first ``rotary_dim`` channels of each head.

    ``layout`` is "neox" (channel j pairs with j + rotary_dim/2) or "interleaved" (2j with 2j+1).
    """

    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    layout: str = "neox"


@dataclass(frozen=True)
class NormSpec(PartSpec):
    dim: int = 0
    eps: float = 1e-6
    # weight enters as (offset + w): 0 for plain RMSNorm, 1 for the "(1 + w)" family
    weight_offset: float = 0.0


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    hidden: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    rope: Optional[RopeSpec] = None
    # a query at position p sees keys j with p - window < j <= p; None = all earlier keys
    window: Optional[int] = None


@dataclass(frozen=True)
class FeedForwardSpec(PartSpec):
    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class BlockSpec:
    """One set of layer weights: pre-norm residual block ``x + mixer(norm(x))``, then
    ``x + ffn(norm(x))``.  ``prefix`` is the tensor-name prefix of the block's weights."""

    prefix: str
    norm_in: NormSpec
    mixer: PartSpec
    norm_post: NormSpec
    feed_forward: PartSpec
    # tensor-name pieces between the block's prefix and each part's own tensor names
    norm_in_name: str = "input_layernorm."
    mixer_name: str = "self_attn."
    norm_post_name: str = "post_attention_layernorm."
    feed_forward_name: str = "mlp."


@dataclass(frozen=True)
class LayerRun:
    """One execution of a block.  ``cache_from`` names an earlier position in the run list whose
    cache this run reads instead of writing its own (None = own cache)."""

    block: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden: int
    embed_name: str
    blocks: Tuple[BlockSpec, ...]
    runs: Tuple[LayerRun, ...]
    final_norm: NormSpec
    final_norm_name: str  # tensor-name prefix of the final norm
    # None = the head reuses the embedding table
    head_name: Optional[str]
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    # standard deviations used by the random-weights mode
    init_std: float = 0.02
    norm_init_std: float = 0.1

    def validate(self) -> None:
        if not self.blocks:
            raise ValueError("a model plan needs at least one block")
        for pos, run in enumerate(self.runs):
            if not (0 <= run.block < len(self.blocks)):
                raise ValueError(f"run {pos} names block {run.block}, but there are {len(self.blocks)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < pos):
                    raise ValueError(f"run {pos} reads the cache of run {run.cache_from}, which is not earlier")
                if self.runs[run.cache_from].cache_from is not None:
                    raise ValueError(f"run {pos} reads the cache of run {run.cache_from}, which owns none")
