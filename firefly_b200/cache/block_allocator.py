"""Free list of cache pages.

The list itself is native code (``csrc/host/block_pool.cc``, built with the host
C++ compiler at first use); this class is its Python face.  Same contract as the
reference's ``BlockAllocator`` (include/firefly/scheduler.h:13-35,
src/scheduler.cc:13-54): ``allocate(n)`` is all-or-nothing, ``free`` gives pages
back, and the list is last-in-first-out, so a page that was just given back is
the next one handed out.  Added: every page is tracked, so freeing a page twice,
freeing a page this allocator never gave out, or losing one is detected.
Page ids run from ``first_id`` (ids below it are reserved, e.g. a scratch page
for padded lanes of a captured graph).
"""
from __future__ import annotations

import ctypes
from typing import Iterable, List, Optional


class PageError(RuntimeError):
    pass


_lib = None


def _native():
    global _lib
    if _lib is None:
        from ..ops.build import load_host_module
        lib = load_host_module("host/block_pool.cc")
        lib.ffh_pool_create.restype = ctypes.c_void_p
        lib.ffh_pool_create.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.ffh_pool_destroy.argtypes = [ctypes.c_void_p]
        lib.ffh_pool_num_free.argtypes = [ctypes.c_void_p]
        lib.ffh_pool_allocate.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        lib.ffh_pool_free.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                      ctypes.POINTER(ctypes.c_int)]
        lib.ffh_pool_check.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        _lib = lib
    return _lib


class BlockAllocator:
    def __init__(self, num_blocks: int, first_id: int = 0):
        if num_blocks < 0:
            raise ValueError("num_blocks must be >= 0")
        self.num_blocks = num_blocks
        self.first_id = first_id
        self._lib = _native()
        self._h = self._lib.ffh_pool_create(num_blocks, first_id)
        if not self._h:
            raise MemoryError("could not create the page pool")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ffh_pool_destroy(h)

    @property
    def num_free(self) -> int:
        return self._lib.ffh_pool_num_free(self._h)

    @property
    def num_held(self) -> int:
        return self.num_blocks - self.num_free

    def can_allocate(self, n: int) -> bool:
        return n <= self.num_free

    def allocate(self, n: int) -> Optional[List[int]]:
        """``n`` pages, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n == 0:
            return []
        buf = (ctypes.c_int * n)()
        rc = self._lib.ffh_pool_allocate(self._h, n, buf)
        if rc == 0:
            return None
        return list(buf)

    def free(self, blocks: Iterable[int]) -> None:
        ids = list(blocks)
        if not ids:
            return
        arr = (ctypes.c_int * len(ids))(*ids)
        bad = ctypes.c_int(0)
        rc = self._lib.ffh_pool_free(self._h, arr, len(ids), ctypes.byref(bad))
        if rc == 1:
            raise PageError(f"page {bad.value} does not belong to this pool "
                            f"[{self.first_id}, {self.first_id + self.num_blocks})")
        if rc == 2:
            raise PageError(f"page {bad.value} freed twice (or never allocated)")

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        bad = ctypes.c_int(0)
        rc = self._lib.ffh_pool_check(self._h, ctypes.byref(bad))
        if rc == 1:
            raise PageError(f"page {bad.value} is on the free list twice")
        if rc == 2:
            raise PageError(f"page {bad.value} is both free and held")
        if rc == 3:
            raise PageError("a page was lost")
