"""The parts a decoder block is put together from, and their registries."""
from .base import (CacheTensor, FeedForward, LayerCache, Mixer, Norm, PagedCacheNeed, Part, PositionEncoding,
                   StepContext, Workspace, build_part, part_class, register_feed_forward,
                   register_mixer, register_norm, register_position_encoding, unregister)
from . import norm, rope, attention, swiglu  # noqa: F401  (register the built-in kinds)
from .block import Block

__all__ = [
    "CacheTensor", "FeedForward", "LayerCache", "Mixer", "Norm", "PagedCacheNeed", "Part", "PositionEncoding",
    "StepContext", "Workspace", "build_part", "part_class", "register_feed_forward",
    "register_mixer", "register_norm", "register_position_encoding", "unregister", "Block",
]
