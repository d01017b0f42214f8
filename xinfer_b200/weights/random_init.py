"""Random-weights mode: from a configuration and a seed to a model folder (config.json and
model.safetensors), or to tensors drawn straight on a device.

The reference always loads files; it has no such mode.  Each tensor is drawn from a generator
seeded by (seed, tensor name), so a tensor's values do not depend on the order in which tensors
are produced or on which other tensors exist.  Linear and embedding weights ~ N(0, std), norm
weights ~ 1 + N(0, norm_std).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Callable, List, Mapping, Optional, Sequence

import torch

from .loader import WeightSpec
from .safetensors_io import write_safetensors


def _seed_of(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def draw(spec: WeightSpec, seed: int, std: float, norm_std: float, dtype: torch.dtype,
         device="cpu") -> torch.Tensor:
    """One tensor.  The stream differs between CPU and CUDA generators: a folder written on the
    CPU and tensors drawn on the GPU with the same seed are different models."""
    g = torch.Generator(device=device)
    g.manual_seed(_seed_of(seed, spec.name))
    shape = tuple(spec.shape)
    if spec.init in ("linear", "embedding"):
        t = torch.randn(shape, generator=g, dtype=torch.float32, device=device).mul_(std)
    elif spec.init == "norm":
        t = torch.randn(shape, generator=g, dtype=torch.float32, device=device).mul_(norm_std).add_(1.0)
    elif spec.init == "zeros":
        t = torch.zeros(shape, dtype=torch.float32, device=device)
    elif spec.init == "ones":
        t = torch.ones(shape, dtype=torch.float32, device=device)
    else:
        raise ValueError(f"weight '{spec.name}' has unknown init kind '{spec.init}'")
    return t.to(dtype)


def write_random_model(model_dir: str, config_dict: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: Optional[float] = None,
                       norm_std: Optional[float] = None,
                       override: Optional[Callable[[str, torch.Tensor], torch.Tensor]] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for the architecture that
    ``config_dict['architectures'][0]`` names.  ``override(name, tensor)`` may return a changed
    tensor (tests use it to plant weights that make one key or one page stand out)."""
    from ..config import config_from_dict
    from ..models.decoder import model_weight_specs

    entry, cfg = config_from_dict(config_dict)
    plan = entry.plan_of(cfg)
    specs = model_weight_specs(plan)
    std = plan.init_std if std is None else std
    norm_std = plan.norm_init_std if norm_std is None else norm_std
    os.makedirs(model_dir, exist_ok=True)
    by_name = {s.name: s for s in specs}

    def produce(name: str) -> torch.Tensor:
        t = draw(by_name[name], seed, std, norm_std, dtype)
        if override is not None:
            t2 = override(name, t)
            if t2 is not None:
                t = t2.to(dtype)
        return t

    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      [(s.name, tuple(s.shape), dtype) for s in specs], produce,
                      metadata={"format": "pt", "seed": str(int(seed))})
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_dict), f, indent=1)
    return model_dir


class RandomWeightStore:
    """Stands where a ``WeightStore`` stands, but draws every tensor on the target device instead
    of reading a file: a model of any size with random weights and nothing written to disk."""

    def __init__(self, specs: Sequence[WeightSpec], seed: int, std: float = 0.02, norm_std: float = 0.1):
        self.specs = {s.name: s for s in specs}
        self.seed = int(seed)
        self.std = std
        self.norm_std = norm_std

    def names(self) -> List[str]:
        return sorted(self.specs)

    def check(self, specs: Sequence[WeightSpec], *, strict: bool = False) -> List[str]:
        from .loader import WeightError
        want = {s.name: tuple(s.shape) for s in specs}
        missing = sorted(n for n in want if n not in self.specs)
        unexpected = sorted(n for n in self.specs if n not in want)
        wrong = [(n, self.specs[n].shape, want[n]) for n in sorted(want) if n in self.specs and tuple(self.specs[n].shape) != want[n]]
        if missing or wrong or (strict and unexpected):
            raise WeightError(missing, unexpected, wrong)
        return unexpected

    def get(self, name: str, device, compute_dtype: torch.dtype, *, operand: bool = False) -> torch.Tensor:
        spec = self.specs[name]
        target = torch.float32 if compute_dtype == torch.float32 else torch.bfloat16
        dev = torch.device(device)
        gen_dev = dev if dev.type == "cuda" else "cpu"
        return draw(spec, self.seed, self.std, self.norm_std, target, device=gen_dev).to(dev).contiguous()

    def close(self) -> None:
        pass
