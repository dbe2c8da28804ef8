"""Free list of cache pages.

Same contract as the reference's ``BlockAllocator`` (include/firefly/scheduler.h:13-35,
src/scheduler.cc:13-54): ``allocate(n)`` is all-or-nothing, ``free`` gives pages
back, and the list is last-in-first-out, so a page that was just given back is
the next one handed out.  Added: every page is tracked, so freeing a page twice,
freeing a page this allocator never gave out, or losing one is detected.
Page ids run from ``first_id`` (ids below it are reserved, e.g. a scratch page
for padded lanes of a captured graph).
"""
from __future__ import annotations

from typing import Iterable, List, Optional


class PageError(RuntimeError):
    pass


class BlockAllocator:
    def __init__(self, num_blocks: int, first_id: int = 0):
        if num_blocks < 0:
            raise ValueError("num_blocks must be >= 0")
        self.num_blocks = num_blocks
        self.first_id = first_id
        # LIFO: the lowest ids are handed out first from a fresh pool
        self._free: List[int] = list(range(first_id + num_blocks - 1, first_id - 1, -1))
        self._held = [False] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_blocks - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int) -> Optional[List[int]]:
        """``n`` pages, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._held[b - self.first_id] = True
        return out

    def free(self, blocks: Iterable[int]) -> None:
        for b in blocks:
            i = b - self.first_id
            if not (0 <= i < self.num_blocks):
                raise PageError(f"page {b} does not belong to this pool "
                                f"[{self.first_id}, {self.first_id + self.num_blocks})")
            if not self._held[i]:
                raise PageError(f"page {b} freed twice (or never allocated)")
            self._held[i] = False
            self._free.append(b)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        seen = set()
        for b in self._free:
            if b in seen:
                raise PageError(f"page {b} is on the free list twice")
            seen.add(b)
            if self._held[b - self.first_id]:
                raise PageError(f"page {b} is both free and held")
        if len(seen) + sum(self._held) != self.num_blocks:
            raise PageError("a page was lost")
