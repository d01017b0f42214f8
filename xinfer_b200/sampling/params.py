"""Per-request sampling options, named as the reference names them
(src/utils/config.rs:797-832; Python constructor src/py/mod.rs:421-463)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union


@dataclass
class SamplingParams:
    # < 1e-7 (or None) selects the most likely token (src/utils/logits_processor.rs:53-59); the
    # reference falls back to 0.7 / top-k 32 / top-p 0.95 when nothing is set
    # (src/core/runner.rs:1843-1854), this engine to greedy
    temperature: Optional[float] = None
    max_tokens: Optional[int] = None
    ignore_eos: bool = False
    top_k: Optional[int] = None      # <= 0 or None: off
    top_p: Optional[float] = None    # outside (0, 1) or None: off
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    # not in the reference: a seed per request, so that a request's samples do not depend on what
    # it is batched with (the reference draws every request from one engine-wide generator,
    # src/utils/logits_processor.rs:20-36)
    seed: Optional[int] = None
    # token ids and / or sequences of token ids that end the request (the reference keeps its stop strings
    # as sequences of ids, src/utils/config.rs:808-809): a sequence is hit when the generated tokens end with
    # it; the token that completes a stop stays out of the output
    stop_token_ids: List[Union[int, Sequence[int]]] = field(default_factory=list)
    session_id: Optional[str] = None

    def validate(self) -> None:
        if self.temperature is not None and not (self.temperature >= 0.0):
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")
        if self.top_p is not None and self.top_p < 0.0:
            raise ValueError(f"top_p must be >= 0, got {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature is None or self.temperature < 1e-7

    @property
    def has_penalties(self) -> bool:
        return bool(self.frequency_penalty) or bool(self.presence_penalty)
