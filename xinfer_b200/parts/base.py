"""Interfaces of the parts a decoder block is put together from, their registries, and the
step context they are handed.  A part knows its own sizes and constants (its spec) and the step's
metadata; it never sees a model configuration or the model it sits in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple, Type

import numpy as np
import torch

from ..config.plan import PartSpec
from ..weights.loader import WeightSpec, WeightStore


class Workspace:
    """Named scratch buffers that live across layers and steps.  A buffer is grown when a larger
    shape is asked for; with ``frozen`` set (while a CUDA graph holds pointers into it) growing
    is an error."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}   # (name, shape, dtype) -> view of the buffer
        self.frozen = False

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._bufs.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if self.frozen and buf is not None:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow while a CUDA graph uses it")
            cap = n if buf is None or buf.dtype != dtype else max(n, buf.numel())
            # zero-filled: rows that padding tokens never write must stay finite
            buf = torch.zeros(max(cap, 1), dtype=dtype, device=self.device)
            self._bufs[name] = buf
            self._views = {k: v for k, v in self._views.items() if k[0] != name}   # they point into the old buffer
        if len(self._views) > 512:
            self._views.clear()
        view = buf[:n].view(*shape)
        self._views[key] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())

    def clear(self) -> None:
        """Zero every buffer (their addresses stay): counters and tickets that kernels keep at zero
        between launches are zero again after a step that did not run to its end."""
        for b in self._bufs.values():
            b.zero_()


@dataclass
class StepContext:
    """Everything a part may know about the running step."""

    dtype: torch.dtype
    device: torch.device
    num_tokens: int            # rows in the activations (including padding tokens)
    num_entries: int           # requests in the batch (including padding entries)
    # device int32 arrays (views into the step's packed metadata)
    token_ids: torch.Tensor    # [T]
    positions: torch.Tensor    # [T]   absolute position of each token in its request
    req_of_token: torch.Tensor # [T]   index of the token's entry in this batch, -1 for padding
    q_start: torch.Tensor      # [B+1] first token of each entry
    start_pos: torch.Tensor    # [B]   tokens already cached for each entry
    slots: torch.Tensor        # [B]   request slot of each entry (row of per-request state)
    logit_rows: torch.Tensor   # [R]   rows whose logits are wanted
    num_logit_rows: int
    tables: List[torch.Tensor] # per cache group: [B, stride] page ids, -1 where none
    strides: List[int]
    err: torch.Tensor          # int32[1] device error word
    workspace: Workspace
    # host copies for parts that loop over entries on the host
    h_q_start: np.ndarray = None
    h_start_pos: np.ndarray = None
    h_slots: np.ndarray = None
    real_tokens: int = 0       # tokens that are not padding
    real_entries: int = 0
    # longest context (start + count) of any entry, and whether every entry brings one token
    max_context: int = 0
    all_single: bool = False
    # the step is (or will be) replayed from a CUDA graph: launch sizes must come from the padded
    # shapes, never from this step's actual lengths
    fixed_shapes: bool = False
    # int32 ids that a sampler left on the device; a token id -1 - i in token_ids stands for sampled[i]
    sampled: Optional[torch.Tensor] = None
    # values parts compute once per step and share between layers
    scratch: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class CacheTensor:
    """One tensor a mixer keeps per cached token: ``shape`` per token, ``dtype`` (None: the
    engine's dtype) and where the in-page token axis sits in the page tensor, which has the shape
    ``(num_pages,) + shape[:token_axis] + (page_size,) + shape[token_axis:]``."""

    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = None
    token_axis: int = 0

    def page_shape(self, num_pages: int, page_size: int) -> Tuple[int, ...]:
        a = self.token_axis
        if not (0 <= a <= len(self.shape)):
            raise ValueError(f"token_axis {a} does not fit a per-token shape {self.shape}")
        return (int(num_pages),) + tuple(self.shape[:a]) + (int(page_size),) + tuple(self.shape[a:])

    def bytes_per_token(self, engine_dtype: torch.dtype) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n * torch.empty((), dtype=self.dtype or engine_dtype).element_size()


@dataclass(frozen=True)
class PagedCacheNeed:
    """What a mixer wants from the paged cache: named tensors per token (keys and values for
    attention, one latent vector for a mixer that caches that, ...), how long tokens are kept
    (``window`` None keeps all) and, if it matters to its kernels, the page size (None: the
    engine's).  Mixers with the same window and page size share a page pool and block tables."""

    tensors: Tuple[Tuple[str, CacheTensor], ...]
    window: Optional[int] = None
    page_size: Optional[int] = None

    @staticmethod
    def keys_and_values(kv_heads: int, head_dim: int, window: Optional[int] = None,
                        page_size: Optional[int] = None) -> "PagedCacheNeed":
        """Keys and values ``[page, kv_head, slot, head_dim]``: a head's page is one contiguous block."""
        t = CacheTensor((int(kv_heads), int(head_dim)), None, 1)
        return PagedCacheNeed((("k", t), ("v", t)), window, page_size)

    def bytes_per_token(self, engine_dtype: torch.dtype) -> int:
        return sum(t.bytes_per_token(engine_dtype) for _, t in self.tensors)


@dataclass
class LayerCache:
    """The pages of one layer run: the mixer's named page tensors (see ``CacheTensor.page_shape``),
    the index of the cache group whose block tables address them, and that group's page size."""

    tensors: Dict[str, torch.Tensor]
    group: int
    page_size: int

    @staticmethod
    def of_keys_and_values(k: torch.Tensor, v: torch.Tensor, group: int, page_size: int) -> "LayerCache":
        return LayerCache({"k": k, "v": v}, group, page_size)

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.tensors[name]


class Part:
    """Base of all parts.  Subclasses set ``kind`` and implement the class method
    ``weight_specs(spec, prefix)`` and the methods ``load`` and ``forward``."""

    kind: str = ""
    # True: ``forward`` takes everything about the step from device tensors of the context (never
    # from its host copies or actual lengths), so a decode step through this part can be captured
    # in a CUDA graph and replayed.  Parts that loop over entries on the host leave it False.
    graph_safe: bool = False

    def __init__(self, spec: PartSpec, prefix: str, dtype: torch.dtype, device):
        self.spec = spec
        self.prefix = prefix
        self.dtype = dtype
        self.device = device

    @classmethod
    def weight_specs(cls, spec: PartSpec, prefix: str) -> List[WeightSpec]:
        return []

    def load(self, store: WeightStore) -> None:
        pass


class Mixer(Part):
    """Mixes information across the tokens of a request.

    ``cache_need()``: pages it wants (or None).  ``state_need()``: fixed-size per-request state,
    a dict name -> (shape, dtype), one row per request slot (or None).
    ``forward(x, ctx, cache, state)`` takes the normed activations ``[T, hidden]`` and returns
    ``[T, hidden]``; it must write this step's keys/values (or state) before reading them, and it
    must give the same result however the request's tokens were cut into steps.
    ``writes_cache`` False means this run reads pages another run wrote.
    """

    def cache_need(self) -> Optional[PagedCacheNeed]:
        return None

    def state_need(self) -> Optional[Dict[str, Tuple[Tuple[int, ...], torch.dtype]]]:
        return None

    def prepare_step(self, ctx: StepContext, cache: Optional[LayerCache]) -> None:
        """Called for every layer run before the step's first kernel: what a mixer wants decided
        once per step from the step's metadata (launch figures, work lists) is decided here."""

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache],
                state: Optional[Dict[str, torch.Tensor]], writes_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """Acts on every token alone: ``forward(x, ctx)`` takes and returns ``[T, hidden]``."""

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    """``forward(out, x, ctx, branch=None, sum_out=None, rows=None)``: out = norm(x (+ branch)),
    optionally on gathered rows; ``sum_out`` receives x + branch."""

    def forward(self, out, x, ctx, branch=None, sum_out=None, rows=None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information for a mixer's queries and keys.  Either it offers rotary tables that
    the attention kernel applies while it writes the cache (``rotary()`` returns them), or it
    rewrites q and k itself in ``apply``."""

    def rotary(self):
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx: StepContext) -> None:
        pass


_REGISTRIES: Dict[str, Dict[str, Type[Part]]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}}


def _register(family: str, kind: str, cls: Type[Part], replace: bool) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} kind '{kind}' is already registered")
    reg[kind] = cls


def register_mixer(kind: str, cls: Type[Mixer], *, replace: bool = False) -> None:
    _register("mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls: Type[FeedForward], *, replace: bool = False) -> None:
    _register("feed_forward", kind, cls, replace)


def register_norm(kind: str, cls: Type[Norm], *, replace: bool = False) -> None:
    _register("norm", kind, cls, replace)


def register_position_encoding(kind: str, cls: Type[PositionEncoding], *, replace: bool = False) -> None:
    _register("position", kind, cls, replace)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def part_class(family: str, kind: str) -> Type[Part]:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise ValueError(f"no {family} of kind '{kind}' is registered (known: {known})") from None


def build_part(family: str, spec: PartSpec, prefix: str, dtype: torch.dtype, device) -> Part:
    return part_class(family, spec.kind)(spec, prefix, dtype, device)
