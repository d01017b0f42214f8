"""Rotary position encoding.  ``inv_freq_j = 1 / theta^(2j / rotary_dim)`` computed in float64
and rounded to float32, angle = position * inv_freq in float32, cos/sin tables in float32
(src/models/layers/rotary_emb.rs:42-62; the reference then rounds the tables to the model dtype,
qwen3.rs:221-231 - here they stay float32 in both precisions).  The tables are applied by the
attention kernel that also norms q/k and writes the cache."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import kernels
from ..config.plan import RopeSpec
from .base import PositionEncoding, register_position_encoding


@dataclass
class RotaryTables:
    cos: torch.Tensor  # [max_positions, rotary_dim / 2] float32
    sin: torch.Tensor
    rotary_dim: int
    interleaved: bool


_TABLE_CACHE = {}


def inv_frequencies(theta: float, rotary_dim: int) -> np.ndarray:
    j = np.arange(0, rotary_dim, 2, dtype=np.float64)
    return (np.float32(1.0) / np.power(np.float64(theta), j / np.float64(rotary_dim)).astype(np.float32)).astype(np.float32)


class Rope(PositionEncoding):
    kind = "rope"
    graph_safe = True

    def __init__(self, spec: RopeSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        if spec.layout not in ("neox", "interleaved"):
            raise ValueError(f"unknown rotary layout '{spec.layout}'")
        self._tables = None

    def rotary(self) -> RotaryTables:
        if self._tables is None:
            s = self.spec
            key = (str(self.device), s.theta, s.rotary_dim, s.max_positions)
            if key not in _TABLE_CACHE:  # layers with the same constants share one table
                half = s.rotary_dim // 2
                inv = torch.from_numpy(inv_frequencies(s.theta, s.rotary_dim)).to(self.device)
                cos = torch.empty((s.max_positions, half), dtype=torch.float32, device=self.device)
                sin = torch.empty_like(cos)
                kernels.rope_table(cos, sin, inv)
                _TABLE_CACHE[key] = (cos, sin)
            cos, sin = _TABLE_CACHE[key]
            self._tables = RotaryTables(cos, sin, s.rotary_dim, s.layout == "interleaved")
        return self._tables


register_position_encoding("rope", Rope)
