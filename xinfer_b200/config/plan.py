"""Typed descriptions of a decoder: what each layer is made of and in which order layers run.

A model is described as data before anything is built:

* a *part spec* per part (mixer, feed-forward, norm, position encoding) carrying every size and
  constant the part needs, so no part ever looks at a model configuration;
* a ``BlockSpec`` per set of weights: its parts and their arrangement as a short program of
  operations (norm, mixer, feed-forward, add) over named activations, so that pre-norm, post-norm,
  sandwich-norm and parallel arrangements, and blocks without a feed-forward, are all data;
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
class BlockOp:
    """One operation of a block's program.  A program works on named activations of shape
    ``[tokens, hidden]``; ``"x"`` is the residual stream that enters and leaves the block, every
    other name is local to the block.

    * ``op="norm"``: ``dst = norm(src)`` with the norm ``spec``;
    * ``op="mixer"`` / ``op="feed_forward"``: ``dst = part(src)`` with the part ``spec``;
    * ``op="add"``: ``dst = dst + src`` (no spec).

    ``name`` is the tensor-name piece between the block's prefix and the part's own tensor names;
    two operations with the same ``op`` and ``name`` are the same part (one set of weights).
    An addition into a value is carried out when that value is next read: by the norm kernel
    that reads it where a norm follows (sum and norm in one pass, the sum in float32), by an
    addition kernel otherwise."""

    op: str
    src: str
    dst: str
    spec: Optional[PartSpec] = None
    name: str = ""


BLOCK_OPS = ("norm", "mixer", "feed_forward", "add")


@dataclass(frozen=True)
class BlockSpec:
    """One set of layer weights and the arrangement of its parts: ``program`` lists the block's
    operations in order.  ``prefix`` is the tensor-name prefix of the block's weights.  A block
    holds at most one mixer (a layer with two is written as two blocks, the first without a
    feed-forward); it may hold none."""

    prefix: str
    program: Tuple[BlockOp, ...]

    def ops_of(self, op: str) -> Tuple[BlockOp, ...]:
        return tuple(o for o in self.program if o.op == op)

    @property
    def mixer(self) -> Optional[PartSpec]:
        ops = self.ops_of("mixer")
        return ops[0].spec if ops else None

    @property
    def feed_forward(self) -> Optional[PartSpec]:
        ops = self.ops_of("feed_forward")
        return ops[0].spec if ops else None

    def norms(self) -> Tuple[NormSpec, ...]:
        return tuple(o.spec for o in self.ops_of("norm"))

    def validate(self) -> None:
        defined = {"x"}
        mixers = set()
        for i, o in enumerate(self.program):
            where = f"block '{self.prefix}' operation {i} ({o.op})"
            if o.op not in BLOCK_OPS:
                raise ValueError(f"{where}: unknown operation; known: {', '.join(BLOCK_OPS)}")
            if o.src not in defined:
                raise ValueError(f"{where}: reads '{o.src}', which no earlier operation has produced")
            if o.op == "add":
                if o.dst not in defined:
                    raise ValueError(f"{where}: adds into '{o.dst}', which no earlier operation has produced")
                if o.spec is not None:
                    raise ValueError(f"{where}: an addition has no part")
                if o.src == o.dst:
                    raise ValueError(f"{where}: adds '{o.src}' to itself")
            else:
                if o.spec is None:
                    raise ValueError(f"{where}: needs a part spec")
                if o.dst == o.src and o.op != "norm":
                    raise ValueError(f"{where}: a part may not write the value it reads")
                defined.add(o.dst)
            if o.op == "mixer":
                mixers.add(o.name)
        if len(mixers) > 1:
            raise ValueError(f"block '{self.prefix}' holds {len(mixers)} mixers; a block holds at most one "
                             f"(write the layer as several blocks)")


def pre_norm_block(prefix: str, norm_in: NormSpec, mixer: PartSpec, norm_post: NormSpec, feed_forward: PartSpec, *,
                   norm_in_name: str = "input_layernorm.", mixer_name: str = "self_attn.",
                   norm_post_name: str = "post_attention_layernorm.", feed_forward_name: str = "mlp.") -> BlockSpec:
    """The pre-norm residual block ``x += mixer(norm_in(x)); x += feed_forward(norm_post(x))``
    (src/models/qwen3.rs:108-134)."""
    return BlockSpec(prefix, (
        BlockOp("norm", "x", "h", norm_in, norm_in_name),
        BlockOp("mixer", "h", "a", mixer, mixer_name),
        BlockOp("add", "a", "x"),
        BlockOp("norm", "x", "h", norm_post, norm_post_name),
        BlockOp("feed_forward", "h", "f", feed_forward, feed_forward_name),
        BlockOp("add", "f", "x"),
    ))


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
    # the embedding rows are multiplied by this (rounded to the activation dtype) before the first block
    embed_scale: Optional[float] = None
    # what happens to the float32 logits after the head: logits *= logit_scale, then
    # logits = logit_softcap * tanh(logits / logit_softcap); None = off
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    # standard deviations used by the random-weights mode
    init_std: float = 0.02
    norm_init_std: float = 0.1

    def validate(self) -> None:
        if not self.blocks:
            raise ValueError("a model plan needs at least one block")
        for b in self.blocks:
            b.validate()
        if self.logit_softcap is not None and not (self.logit_softcap > 0):
            raise ValueError(f"logit_softcap must be positive, got {self.logit_softcap}")
        for pos, run in enumerate(self.runs):
            if not (0 <= run.block < len(self.blocks)):
                raise ValueError(f"run {pos} names block {run.block}, but there are {len(self.blocks)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < pos):
                    raise ValueError(f"run {pos} reads the cache of run {run.cache_from}, which is not earlier")
                if self.runs[run.cache_from].cache_from is not None:
                    raise ValueError(f"run {pos} reads the cache of run {run.cache_from}, which owns none")
