"""The page allocator as a Python object (the native BlockAllocator)."""
from __future__ import annotations

import ctypes

from .native import CacheError, checked, last_error, lib


class BlockAllocator:
    """FIFO allocator of page ids 0..total-1
    (crates/cellm-cache/src/allocator.rs:11-90)."""

    def __init__(self, total: int):
        self._h = lib().cellm_alloc_create(int(total))
        if not self._h:
            raise CacheError(last_error())
        self.total = int(total)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().cellm_alloc_destroy(self._h)
            self._h = None

    def alloc(self):
        p = lib().cellm_alloc_alloc(self._h)
        return None if p < 0 else p

    def alloc_n(self, n: int):
        buf = (ctypes.c_int * max(n, 1))()
        ok = checked(lib().cellm_alloc_alloc_n(self._h, n, buf))
        return list(buf[:n]) if ok else None

    def free(self, page: int) -> None:
        checked(lib().cellm_alloc_free(self._h, int(page)))

    @property
    def free_count(self) -> int:
        return lib().cellm_alloc_free_count(self._h)

    def is_free(self, page: int) -> bool:
        return bool(checked(lib().cellm_alloc_is_free(self._h, int(page))))
