"""One layer: the parts of a ``BlockSpec`` and the executor of its program.

A block's arrangement is data (``BlockSpec.program``): operations ``norm``, ``mixer``,
``feed_forward`` and ``add`` over named activations, ``"x"`` being the residual stream.  The
reference wires its one arrangement by hand, ``x + mixer(norm(x))`` then ``x + mlp(norm(x))``
(src/models/qwen3.rs:108-134), and fuses each residual sum with the norm after it
(src/models/layers/others.rs:48-62).

Here an addition is carried out when its sum is next read.  Where a norm reads it, the norm
kernel forms the sum in float32, stores it and norms it in one pass - also across the block
boundary: the last addition of a block waits in the ``Stream`` that the next block (or the
decoder's final norm) receives.  Where a mixer or a feed-forward runs next, an addition kernel
runs first (for every waiting addition: the part may reuse the buffer an addend lives in).
The pre-norm block therefore launches exactly the kernels a hand-written one would.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels, tracing
from ..config.plan import BlockSpec
from ..weights.loader import WeightSpec
from .base import LayerCache, Part, StepContext, build_part, part_class

_FAMILY = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}


class Stream:
    """The residual stream between blocks: its tensor and the branches still to be added to it."""

    __slots__ = ("x", "pending")

    def __init__(self, x: torch.Tensor, pending: Optional[List[torch.Tensor]] = None):
        self.x = x
        self.pending: List[torch.Tensor] = pending or []

    def settle(self, keep_last: bool = False) -> Optional[torch.Tensor]:
        """Carry out the waiting additions; with ``keep_last`` the last one is handed back for a
        norm kernel to fuse."""
        last = self.pending.pop() if (keep_last and self.pending) else None
        for b in self.pending:
            kernels.add(self.x, self.x, b)
        self.pending = []
        return last


class Block:
    def __init__(self, spec: BlockSpec, dtype, device):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.parts: Dict[Tuple[str, str], Part] = {}
        for o in spec.program:
            if o.op == "add":
                continue
            key = (o.op, o.name)
            if key not in self.parts:
                self.parts[key] = build_part(_FAMILY[o.op], o.spec, spec.prefix + o.name, dtype, device)
        mixers = [p for (op, _), p in self.parts.items() if op == "mixer"]
        self.mixer = mixers[0] if mixers else None

    @staticmethod
    def weight_specs(spec: BlockSpec) -> List[WeightSpec]:
        out: List[WeightSpec] = []
        seen = set()
        for o in spec.program:
            if o.op == "add" or (o.op, o.name) in seen:
                continue
            seen.add((o.op, o.name))
            out += part_class(_FAMILY[o.op], o.spec.kind).weight_specs(o.spec, spec.prefix + o.name)
        return out

    def all_parts(self) -> List[Part]:
        return list(self.parts.values())

    def load(self, store) -> None:
        for part in self.parts.values():
            part.load(store)

    def forward(self, stream: Stream, ctx: StepContext, cache: Optional[LayerCache], state, writes_cache: bool) -> Stream:
        """Runs the program on the residual stream; returns the stream with the additions that
        still wait."""
        T, H = stream.x.shape
        ws = ctx.workspace
        vals: Dict[str, torch.Tensor] = {"x": stream.x}
        waiting: Dict[str, List[torch.Tensor]] = {"x": stream.pending}

        def read(name: str) -> torch.Tensor:
            """The value with every addition into it carried out."""
            t = vals[name]
            for b in waiting.pop(name, ()):
                kernels.add(t, t, b)
            return t

        def settle_all() -> None:
            # a part is about to run and may reuse the buffer that a waiting addend lives in
            for name in list(waiting):
                read(name)

        for o in self.spec.program:
            if o.op == "add":
                waiting.setdefault(o.dst, []).append(read(o.src))
                continue
            part = self.parts[(o.op, o.name)]
            if o.op == "norm":
                src = vals[o.src]
                adds = waiting.pop(o.src, [])
                for b in adds[:-1]:
                    kernels.add(src, src, b)
                out = ws.get("block." + o.dst, tuple(src.shape), self.dtype)
                if any(out.data_ptr() == t.data_ptr() for t in (src, *adds)):
                    # a norm back into its own input (or over its addend) gets a buffer of its own
                    out = ws.get("block." + o.dst + "'", tuple(src.shape), self.dtype)
                if tracing.ENABLED:
                    tracing.push("norm")
                if adds:
                    part.forward(out, src, ctx, branch=adds[-1], sum_out=src)
                else:
                    part.forward(out, src, ctx)
                if tracing.ENABLED:
                    tracing.pop()
            else:
                settle_all()
                if tracing.ENABLED:
                    tracing.push(o.op + ":" + part.kind)
                if o.op == "mixer":
                    out = part.forward(vals[o.src], ctx, cache, state, writes_cache)
                else:
                    out = part.forward(vals[o.src], ctx)
                if tracing.ENABLED:
                    tracing.pop()
            waiting.pop(o.dst, None)      # additions that waited for the value this one replaces are void
            vals[o.dst] = out
        # additions into block-local values that nothing read are void; the stream's wait for its next reader
        return Stream(vals["x"], waiting.get("x", []))
