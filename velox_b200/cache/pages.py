"""Page ids and state slots: the host-side bookkeeping of the cache.

`PageAllocator` follows the reference's free list and reference counts
(src/paged/pages.rs:113, 173-242): a stack of free ids made so that page 0 is
handed out first, `alloc(n)` all or nothing, a count per page that `free`
lowers and that returns the page to the stack at zero.  Where the reference only
warns about a bad id or a second free (src/paged/pages.rs:205-212), these raise:
a page freed twice would be handed to two requests.
"""
from __future__ import annotations

from typing import Iterable, List, Optional


class CacheAccountingError(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._refs: List[int] = [0] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        """n pages with count 1, or None (and nothing taken) if fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate %d pages" % n)
        if len(self._free) < n:
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._refs[p] != 0:
                raise CacheAccountingError("page %d was on the free list with count %d" % (p, self._refs[p]))
            self._refs[p] = 1
        return out

    def incref(self, pages: Iterable[int]) -> None:
        for p in pages:
            self._check(p)
            if self._refs[p] < 1:
                raise CacheAccountingError("page %d is free and cannot be shared" % p)
            self._refs[p] += 1

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            self._check(p)
            if self._refs[p] < 1:
                raise CacheAccountingError("page %d freed twice" % p)
            self._refs[p] -= 1
            if self._refs[p] == 0:
                self._free.append(p)

    def refcount(self, page: int) -> int:
        self._check(page)
        return self._refs[page]

    def _check(self, p: int) -> None:
        if not 0 <= p < self.num_pages:
            raise CacheAccountingError("page id %r is outside the pool of %d" % (p, self.num_pages))


class SlotAllocator:
    """Slots for per-request state of fixed size; the lowest free slot first."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("a slot pool needs at least one slot")
        self.num_slots = int(num_slots)
        self._free: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._held = [False] * self.num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._held[s] = True
        return s

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheAccountingError("state slot %r is not held" % slot)
        self._held[slot] = False
        self._free.append(slot)
