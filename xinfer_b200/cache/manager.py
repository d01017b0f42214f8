"""The cache manager: pages of keys and values with a block table per request, one pool per group
of layers with the same needs, and slots for fixed-size per-request state.

The bookkeeping is native (csrc/host/cache_manager.cpp); this module is its Python face and owns
nothing but the handle.  Device storage for the pages belongs to the layers' caches
(xinfer_b200/cache/storage.py); a page id of a group addresses that page in every layer of the
group, as in the reference (src/utils/kvcache_allocator.rs:1641-1654).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence


from ..native import host_lib


@dataclass(frozen=True)
class CacheGroup:
    """Layers whose caches grow alike: same page size, same retention (all keys or a window)."""

    page_size: int
    num_pages: int
    window: Optional[int] = None  # None: keep every key


class CacheError(RuntimeError):
    pass


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroup], max_requests: int):
        if not groups:
            raise CacheError("a cache manager needs at least one group (use a 1-page group for models without caches)")
        self.groups = list(groups)
        self.max_requests = int(max_requests)
        lib = host_lib()
        n = len(self.groups)
        arr = ctypes.c_int * n
        self._lib = lib
        self._h = lib.xb_cm_create(
            n, arr(*[g.page_size for g in self.groups]), arr(*[g.num_pages for g in self.groups]),
            arr(*[(g.window or 0) for g in self.groups]), self.max_requests)
        if not self._h:
            raise CacheError(f"invalid cache groups {self.groups} / max_requests {max_requests}")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.xb_cm_destroy(h)

    @property
    def handle(self):
        return self._h

    # ---- requests --------------------------------------------------------------------------------
    def open_request(self) -> int:
        slot = self._lib.xb_cm_open(self._h)
        if slot < 0:
            raise CacheError(f"all {self.max_requests} request slots are taken")
        return slot

    def close_request(self, slot: int) -> None:
        if not self._lib.xb_cm_close(self._h, slot):
            raise CacheError(f"slot {slot} is not live (closed twice?)")

    def is_live(self, slot: int) -> bool:
        return bool(self._lib.xb_cm_is_live(self._h, slot))

    def length(self, slot: int) -> int:
        n = self._lib.xb_cm_length(self._h, slot)
        if n < 0:
            raise CacheError(f"slot {slot} is not live")
        return n

    def can_extend(self, slot: int, new_len: int) -> bool:
        return bool(self._lib.xb_cm_can_extend(self._h, slot, new_len))

    def extend(self, slot: int, new_len: int) -> bool:
        """Take the pages for tokens [length, new_len) in every group; all or nothing."""
        return bool(self._lib.xb_cm_extend(self._h, slot, new_len))

    def advance(self, slot: int, new_len: int) -> None:
        if not self._lib.xb_cm_advance(self._h, slot, new_len):
            raise CacheError(f"cannot advance slot {slot} to {new_len} tokens (not live, shorter than before, or pages missing)")

    # ---- inspection ------------------------------------------------------------------------------
    def free_pages(self, group: int = 0) -> int:
        return self._lib.xb_cm_free_pages(self._h, group)

    def live_requests(self) -> int:
        return self._lib.xb_cm_live_requests(self._h)

    def table(self, slot: int, group: int = 0) -> List[int]:
        n = self._lib.xb_cm_table_size(self._h, slot, group)
        if n < 0:
            raise CacheError(f"slot {slot} is not live")
        buf = (ctypes.c_int32 * max(n, 1))()
        self._lib.xb_cm_copy_table(self._h, slot, group, buf, n)
        return list(buf[:n])

    def log_freed(self, on: bool = True) -> None:
        """Debug aid: record every page that goes back to a pool, for ``drain_freed``."""
        self._lib.xb_cm_log_freed(self._h, int(bool(on)))

    def drain_freed(self) -> List[tuple]:
        """(group, page) of the pages that went back since the last call (with ``log_freed`` on)."""
        import numpy as np
        out: List[tuple] = []
        g = np.zeros(256, dtype=np.int32)
        p = np.zeros(256, dtype=np.int32)
        while True:
            n = self._lib.xb_cm_drain_freed(self._h, g.ctypes.data, p.ctypes.data, 256)
            out += list(zip(g[:n].tolist(), p[:n].tolist()))
            if n < 256:
                return out

    def check_consistent(self) -> None:
        why = ctypes.create_string_buffer(256)
        if not self._lib.xb_cm_consistent(self._h, why, 256):
            raise CacheError("cache bookkeeping is inconsistent: " + why.value.decode())


class StateSlots:
    """Fixed-size per-request state, one row per request slot.

    A part that keeps state of its own (a recurrent mixer, a sampler counter) asks for a table
    ``[max_requests, *shape]``; the row of a request is its slot in the cache manager.  The
    reference indexes recurrent state the same way through a slot mapping built per step
    (src/core/runner.rs:252-289).  Rows are cleared when a request opens.
    """

    def __init__(self, max_requests: int, device):
        self.max_requests = max_requests
        self.device = device
        self.tables = {}

    def add(self, name: str, shape, dtype):
        import torch
        if name in self.tables:
            raise CacheError(f"state table '{name}' exists already")
        t = torch.zeros((self.max_requests, *shape), dtype=dtype, device=self.device)
        self.tables[name] = t
        return t

    def clear_slot(self, slot: int) -> None:
        for t in self.tables.values():
            t[slot].zero_()
