"""NVTX ranges around steps and kernel classes, behind a flag.

``XINFER_B200_NVTX=1`` in the environment (or ``enable()``) makes the engine push a range per step
("prefill", "decode" or "mixed", with its token and request counts) and, inside it, per class of
work ("embedding", "norm", "mixer:<kind>", "feed_forward:<kind>", "head", "sample"), so that a
timeline of a profiler shows where a step's time goes.  Off by default: the call sites test one
module attribute and do nothing else.  The reference marks its prefill and decode steps the same
way (src/core/runner.rs:1019-1020, 1214-1215).
"""
from __future__ import annotations

import os
from typing import Callable, Optional

ENABLED = os.environ.get("XINFER_B200_NVTX", "0") == "1"

_push: Optional[Callable[[str], object]] = None
_pop: Optional[Callable[[], object]] = None


def _backend():
    global _push, _pop
    if _push is None:
        import torch
        _push, _pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop
    return _push, _pop


def enable(flag: bool = True, push: Optional[Callable[[str], object]] = None,
           pop: Optional[Callable[[], object]] = None) -> None:
    """Switch the ranges on or off; ``push`` / ``pop`` replace NVTX (tests record the calls)."""
    global ENABLED, _push, _pop
    ENABLED = bool(flag)
    _push, _pop = push, pop


def push(name: str) -> None:
    if ENABLED:
        _backend()[0](name)


def pop() -> None:
    if ENABLED:
        _backend()[1]()


def step_kind(counts) -> str:
    """"decode" when every entry brings one token, "prefill" when none does, else "mixed"."""
    ones = sum(1 for c in counts if c == 1)
    if ones == len(counts):
        return "decode"
    return "prefill" if ones == 0 else "mixed"
