"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

The reference spreads this over a string match (src/utils/mod.rs:2355-2469), a constructor macro
(src/core/mod.rs:131-150) and a dispatch enum (src/core/runner.rs:93-113).  Here an entry is a
config class plus a function from that config to a ``ModelPlan``; the generic decoder builds any
plan, so adding an architecture means adding one entry (and parts, if it needs new ones).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .errors import ConfigError
from .plan import ModelPlan


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    plan_of: Callable[[Any], ModelPlan]


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, config_from_dict: Callable[[Mapping[str, Any]], Any],
                          plan_of: Callable[[Any], ModelPlan], *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_from_dict, plan_of)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_entry(name: str) -> ArchitectureEntry:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture '{name}'; registered: {', '.join(known_architectures())}") from None


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in '{model_dir}'")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw


def config_from_dict(raw: Mapping[str, Any]):
    """Choose the architecture by ``architectures`` (exactly one entry, as the reference requires,
    src/core/engine.rs:166-169) and return (entry, typed config)."""
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"config key 'architectures' must be a list with exactly one name, got {archs!r}")
    entry = architecture_entry(archs[0])
    return entry, entry.config_from_dict(raw)


def load_config(model_dir: str):
    return config_from_dict(read_config_json(model_dir))


def _register_builtin() -> None:
    # the one architecture this engine ships; others are added by their own modules the same way
    from .qwen3 import Qwen3Config
    register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.from_dict, lambda c: c.plan())


_register_builtin()
