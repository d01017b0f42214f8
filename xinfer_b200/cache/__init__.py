"""The cache manager: paged keys/values per layer group, block tables, per-request state slots."""
from .manager import CacheError, CacheGroup, CacheManager, StateSlots

__all__ = ["CacheError", "CacheGroup", "CacheManager", "StateSlots"]
