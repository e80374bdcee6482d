"""Page ids and state slots: the host-side bookkeeping of the cache.

`PageAllocator` follows the reference's free list and reference counts
(src/paged/pages.rs:113, 173-242): a stack of free ids made so that page 0 is
handed out first, `alloc(n)` all or nothing, a count per page that `free`
lowers and that returns the page to the stack at zero.  Where the reference only
warns about a bad id or a second free (src/paged/pages.rs:205-212), these raise:
a page freed twice would be handed to two requests.

The pools themselves live in the host library (`csrc/host/pages.hpp`); these
classes own one, or look into one that a `CacheManager` owns.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Iterable, List, Optional

from .. import native
from ..native import CacheAccountingError  # noqa: F401  (part of this module's interface)


class PageAllocator:
    def __init__(self, num_pages: int, _borrowed: Optional[int] = None, _owner=None):
        self._lib = native.library()
        # a pool inside a cache manager's books lives as long as that manager: a weak
        # proxy to it turns a use after its end into a ReferenceError, not a bad pointer
        self._owner = weakref.proxy(_owner) if _owner is not None else None
        if _borrowed is not None:
            self._pool, self._owned = ctypes.c_void_p(_borrowed), False
        else:
            if num_pages <= 0:
                raise ValueError("a page pool needs at least one page")
            self._pool, self._owned = ctypes.c_void_p(self._lib.vxh_pages_create(int(num_pages))), True
        self.num_pages = self._lib.vxh_pages_num_pages(self._pool)

    def __del__(self):
        if getattr(self, "_owned", False) and self._pool:
            self._lib.vxh_pages_destroy(self._pool)
            self._pool = None

    def _alive(self) -> None:
        if self._owner is not None:
            self._owner.page_size  # raises ReferenceError once the manager is gone

    @property
    def num_free(self) -> int:
        self._alive()
        return self._lib.vxh_pages_num_free(self._pool)

    def alloc(self, n: int) -> Optional[List[int]]:
        """n pages with count 1, or None (and nothing taken) if fewer are free."""
        self._alive()
        if n < 0:
            raise ValueError("cannot allocate %d pages" % n)
        out = (ctypes.c_int * max(n, 1))()
        return list(out[:n]) if native.check(self._lib.vxh_pages_alloc(self._pool, n, out)) else None

    def incref(self, pages: Iterable[int]) -> None:
        self._alive()
        arr = native.int_array(pages)
        native.check(self._lib.vxh_pages_incref(self._pool, arr, len(arr)))

    def free(self, pages: Iterable[int]) -> None:
        self._alive()
        arr = native.int_array(pages)
        native.check(self._lib.vxh_pages_free(self._pool, arr, len(arr)))

    def refcount(self, page: int) -> int:
        self._alive()
        return native.check(self._lib.vxh_pages_refcount(self._pool, int(page)))

    def free_list(self) -> List[int]:
        """The free ids, the next one handed out last."""
        self._alive()
        out = (ctypes.c_int * self.num_pages)()
        n = self._lib.vxh_pages_free_list(self._pool, out, self.num_pages)
        return list(out[:n])


class SlotAllocator:
    """Slots for per-request state of fixed size; the lowest free slot first."""

    def __init__(self, num_slots: int, _borrowed: Optional[int] = None, _owner=None):
        self._lib = native.library()
        self._owner = weakref.proxy(_owner) if _owner is not None else None
        if _borrowed is not None:
            self._pool, self._owned = ctypes.c_void_p(_borrowed), False
        else:
            if num_slots <= 0:
                raise ValueError("a slot pool needs at least one slot")
            self._pool, self._owned = ctypes.c_void_p(self._lib.vxh_slots_create(int(num_slots))), True
        self.num_slots = self._lib.vxh_slots_num_slots(self._pool)

    def __del__(self):
        if getattr(self, "_owned", False) and self._pool:
            self._lib.vxh_slots_destroy(self._pool)
            self._pool = None

    def _alive(self) -> None:
        if self._owner is not None:
            self._owner.page_size

    @property
    def num_free(self) -> int:
        self._alive()
        return self._lib.vxh_slots_num_free(self._pool)

    def alloc(self) -> Optional[int]:
        self._alive()
        s = self._lib.vxh_slots_alloc(self._pool)
        return None if s < 0 else s

    def free(self, slot: int) -> None:
        self._alive()
        native.check(self._lib.vxh_slots_free(self._pool, int(slot)))
