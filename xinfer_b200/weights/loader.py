"""Weights by tensor name.

Every part declares the tensors it needs as ``WeightSpec`` (full name, shape, how the
random-weights mode draws it).  ``WeightStore.check`` compares the declared set with what the
files hold and raises ONE error that lists missing tensors, unexpected tensors and wrong shapes.
Tensors the model does not declare are no error by themselves (a checkpoint may carry a spare
head beside a tied one, or position buffers): they are listed in a warning and in
``WeightStore.unexpected``; ``strict=True`` makes them fatal.
``WeightStore.get`` hands a tensor to a part on the target device:

* 16-bit floats arrive as bfloat16 (float32 when the engine runs in float32);
* a tensor stored in 32-bit floats stays float32 - unless the part asks for it as an operand of
  the engine's matrix products (``operand=True``: projection, embedding and head matrices), which
  take the engine's dtype whatever the file holds, as the reference casts them at load;
* integer tables arrive as int32.

The reference resolves names through a prefix-pushing handle over the mapped files
(src/models/layers/mod.rs:170-194) and casts linear weights to the model dtype at load
(src/models/layers/linear.rs:133-138); norm weights are held in float32 (src/models/qwen3.rs:83).
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, find_weight_files


class WeightError(ValueError):
    """The files do not hold exactly the tensors the model declares."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["model weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unsupported dtype ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: {dt}" for n, dt in self.wrong_dtype))
        super().__init__("\n".join(lines))


class UnexpectedWeightsWarning(UserWarning):
    """The files hold tensors that the model does not declare; they are not loaded."""


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    # how the random-weights mode draws it: "linear", "embedding" (both N(0, std)),
    # "norm" (1 + N(0, norm_std)), "zeros", "ones"
    init: str = "linear"


_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightStore:
    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files = [SafetensorsFile(p) for p in find_weight_files(model_dir)]
        self.index: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.entries:
                self.index[name] = f
        self.unexpected: List[str] = []   # filled by check(): tensors of the files that no part declared

    def names(self) -> List[str]:
        return sorted(self.index)

    def check(self, specs: Sequence[WeightSpec], *, strict: bool = False) -> List[str]:
        """Raise one ``WeightError`` for missing tensors, wrong shapes and unsupported dtypes (it
        lists the unexpected tensors too).  Unexpected tensors alone are returned and warned about,
        or raised for with ``strict``."""
        want = {}
        for s in specs:
            want[s.name] = tuple(s.shape)
        missing = sorted(n for n in want if n not in self.index)
        unexpected = sorted(n for n in self.index if n not in want)
        wrong_shape, wrong_dtype = [], []
        for n, shape in sorted(want.items()):
            f = self.index.get(n)
            if f is None:
                continue
            e = f.entries[n]
            if tuple(e.shape) != shape:
                wrong_shape.append((n, e.shape, shape))
            if e.dtype not in _FLOATS and e.dtype not in _INTS:
                wrong_dtype.append((n, str(e.dtype)))
        if missing or wrong_shape or wrong_dtype or (strict and unexpected):
            raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)
        self.unexpected = unexpected
        if unexpected:
            shown = ", ".join(unexpected[:8]) + (f", ... ({len(unexpected) - 8} more)" if len(unexpected) > 8 else "")
            warnings.warn(f"{len(unexpected)} tensor(s) of '{self.model_dir}' are not part of the model and are not "
                          f"loaded: {shown}", UnexpectedWeightsWarning, stacklevel=2)
        return unexpected

    def raw(self, name: str) -> torch.Tensor:
        """The stored tensor on the CPU, in its stored dtype."""
        return self.index[name].tensor(name)

    def get(self, name: str, device, compute_dtype: torch.dtype, *, operand: bool = False) -> torch.Tensor:
        """``operand``: the tensor is an operand of the engine's matrix products and takes
        ``compute_dtype`` whatever it was stored in (src/models/layers/linear.rs:133-138)."""
        t = self.raw(name)
        if t.dtype in _INTS:
            return t.to(device=device, dtype=torch.int32)
        if compute_dtype == torch.float32 or (not operand and t.dtype in (torch.float32, torch.float64)):
            target = torch.float32
        else:
            target = torch.bfloat16
        return t.to(device=device).to(target).contiguous()

    def close(self) -> None:
        for f in self.files:
            f.close()
