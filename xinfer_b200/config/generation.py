"""Default sampling options of a model folder and of an engine.

The reference reads ``generation_config.json`` beside ``config.json`` (src/utils/mod.rs:1868-1876,
fields src/utils/config.rs:1022-1038), lets the engine's own ``generation_cfg`` win field by field
(src/utils/mod.rs:2577-2599), fills what a request leaves unset from the result
(src/core/engine.rs:680-692) and joins its EOS ids with those of ``config.json``
(src/utils/config.rs:360-375).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Optional, Tuple

from .errors import ConfigError

FILE_NAME = "generation_config.json"
_SAMPLING_FIELDS = ("temperature", "top_p", "top_k", "frequency_penalty", "presence_penalty")


@dataclass
class GenerationConfig:
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "GenerationConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"{FILE_NAME} must hold a JSON object, got {type(raw).__name__}")

        def number(key, kind):
            v = raw.get(key)
            if v is None:
                return None
            if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and v != int(v)):
                raise ConfigError(f"{FILE_NAME}: key '{key}' must be {'an integer' if kind is int else 'a number'}, got {v!r}")
            return kind(v)

        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{FILE_NAME}: key 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
        return cls(temperature=number("temperature", float), top_p=number("top_p", float), top_k=number("top_k", int),
                   frequency_penalty=number("frequency_penalty", float), presence_penalty=number("presence_penalty", float),
                   bos_token_id=number("bos_token_id", int), eos_token_id=eos_ids)

    @classmethod
    def load(cls, folder: str) -> Optional["GenerationConfig"]:
        """The folder's generation_config.json, or None where it has none."""
        path = os.path.join(folder, FILE_NAME)
        if not os.path.isfile(path):
            return None
        try:
            with open(path) as f:
                raw = json.load(f)
        except (OSError, ValueError) as e:
            raise ConfigError(f"cannot read {path}: {e}") from e
        return cls.from_dict(raw)

    def over(self, other: Optional["GenerationConfig"]) -> "GenerationConfig":
        """This one's fields where they are set, ``other``'s elsewhere."""
        if other is None:
            return self
        merged = {f.name: getattr(self, f.name) if getattr(self, f.name) not in (None, ()) else getattr(other, f.name)
                  for f in fields(self)}
        return GenerationConfig(**merged)

    def fill(self, params):
        """A copy of a request's sampling options with what it left unset taken from here."""
        import dataclasses
        unset = {k: getattr(self, k) for k in _SAMPLING_FIELDS if getattr(params, k) is None and getattr(self, k) is not None}
        return dataclasses.replace(params, **unset) if unset else params


def join_eos(model_ids: Tuple[int, ...], generation: Optional[GenerationConfig]) -> Tuple[int, ...]:
    """config.json's EOS ids followed by those that only generation_config.json names."""
    ids = list(model_ids)
    for e in (generation.eos_token_id if generation is not None else ()):
        if e not in ids:
            ids.append(e)
    return tuple(ids)
