"""The cache manager: pages of keys and values with a block table per request,
in groups of layers with the same needs, and slots for fixed-size state.

The manager is told, for every place of the model's running order, what the
mixer there needs (a layer that runs twice has two places and two caches).
What lies in a page or a slot is the business of the need's `CacheKind`
(`cache/kinds.py`: keys and values in pages, fixed-size state, and whatever kind
is registered besides).  Places that ask for the same paged need (for keys and
values: kv heads, head size, window) form a group.  A group has its own page
pool, storage laid out by its kind, and its own block table per request: entry i
is the page that holds positions [i*S, (i+1)*S), or -1.  Pages are taken when a
step needs them (`reserve`), not for the worst case at admission as the
reference does (src/paged/scheduler.rs:255).  They are given back when the
request ends, and in a group with a window as soon as every position of a page
lies before the window of the next query; the freed page is the next one handed
out.

Layers whose mixers ask for a slot kind (`FixedState`) get one tensor [slots, *shape] each;
a request holds one slot id from admission to its end, in every such layer.
Qwen3 has no such layer; the slot is assigned all the same.

The bookkeeping is host-only and runs without a device (`device=None`).  It is
kept by the host library (`csrc/host/cache_book.hpp`): pools, block tables, slots
and lengths live there, where the scheduler and the step builders read them
directly; this class owns the device storage and answers questions about the
books.
"""
from __future__ import annotations

import ctypes
import weakref
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Mapping, Optional, Sequence

import torch

from .. import native
from ..native import OutOfPages  # noqa: F401  (part of this module's interface)
from .kinds import CacheKind, LayerCache, cache_kind
from .pages import CacheAccountingError, PageAllocator, SlotAllocator


@dataclass
class CacheGroup:
    spec: object               # the paged need that the group's layers share
    kind: CacheKind
    layers: List[int]
    allocator: PageAllocator
    storage: Optional[torch.Tensor] = None  # laid out by the kind; first dimension: the group's layers

    @property
    def window(self) -> int:
        return self.kind.window(self.spec)


@dataclass
class RequestCache:
    """A request's books as they were when it was looked up."""
    slot: int
    length: int = 0  # positions whose keys/values (or state) are in the cache
    tables: List[List[int]] = field(default_factory=list)  # per group


class _Requests(Mapping):
    """`manager.requests`: request id -> `RequestCache` (a copy made at the lookup)."""

    def __init__(self, manager: "CacheManager"):
        self._m = weakref.proxy(manager)  # (the manager holds this view: no cycle, so it ends when dropped)

    def __getitem__(self, request_id) -> RequestCache:
        m = self._m
        h = m._handle(request_id, create=False)
        if h is None or not m._lib.vxh_cache_has(m._book, h):
            raise KeyError(request_id)
        tables = []
        buf = (ctypes.c_int * m.max_blocks)()
        for g in range(len(m.groups)):
            n = native.check(m._lib.vxh_cache_table(m._book, h, g, buf, m.max_blocks))
            tables.append(list(buf[:n]))
        return RequestCache(m._lib.vxh_cache_slot(m._book, h), int(m._lib.vxh_cache_length(m._book, h)), tables)

    def __iter__(self) -> Iterator:
        m = self._m
        n = m._lib.vxh_cache_num_requests(m._book)
        ids = (ctypes.c_int64 * max(n, 1))()
        m._lib.vxh_cache_request_ids(m._book, ids, n)
        return iter([m._names.get(h, h) for h in ids[:n]])

    def __len__(self) -> int:
        return int(self._m._lib.vxh_cache_num_requests(self._m._book))


class CacheManager:
    def __init__(self, cache_specs: Sequence, cache_of: Sequence[Optional[int]], page_size: int, num_pages: int,
                 max_requests: int, max_blocks: int, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None, poison: bool = False):
        self.page_size, self.max_blocks = int(page_size), int(max_blocks)
        self.dtype, self.device = dtype, device
        self.groups: List[CacheGroup] = []
        self._layers: List[LayerCache] = []
        self._state_layers: List[int] = []
        by_spec: Dict[object, int] = {}
        n_layers = len(cache_specs)
        layer_group = [-1] * n_layers
        specs_of_groups: List[object] = []
        layers_of_groups: List[List[int]] = []
        kinds = [None if spec is None else cache_kind(spec) for spec in cache_specs]
        for i, spec in enumerate(cache_specs):
            if spec is not None and kinds[i].paged:
                if spec not in by_spec:
                    by_spec[spec] = len(specs_of_groups)
                    specs_of_groups.append(spec)
                    layers_of_groups.append([])
                layer_group[i] = by_spec[spec]
                layers_of_groups[by_spec[spec]].append(i)
        # the books: pools, block tables, slots and lengths live in the host library
        self._lib = native.library()
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        windows = native.int_array([cache_kind(s).window(s) for s in specs_of_groups])
        self._book = ctypes.c_void_p(self._lib.vxh_cache_create(len(specs_of_groups), windows, self.page_size,
                                                                int(num_pages), int(max_requests), self.max_blocks))
        if not self._book:
            raise ValueError("page size, pages, requests and blocks per request must be positive")
        self.slots = SlotAllocator(0, _borrowed=self._lib.vxh_cache_slots(self._book), _owner=self)
        for g, (spec, layers) in enumerate(zip(specs_of_groups, layers_of_groups)):
            self.groups.append(CacheGroup(spec, cache_kind(spec), layers,
                                          PageAllocator(0, _borrowed=self._lib.vxh_cache_pool(self._book, g), _owner=self)))
        # request ids: non-negative integers are their own handle in the library
        # (the scheduler's ids are such), anything else gets a negative one
        self._handles: Dict[object, int] = {}
        self._names: Dict[int, object] = {}
        self._next_handle = -1
        self.requests = _Requests(self)
        for g in self.groups:
            if device is not None:
                g.storage = g.kind.allocate(g.spec, len(g.layers), num_pages, self.page_size, dtype, device)
                if poison and g.storage.is_floating_point():
                    g.storage.fill_(float("nan"))
                else:
                    g.storage.zero_()
        self._state_kinds: Dict[int, CacheKind] = {}
        for i, spec in enumerate(cache_specs):
            if spec is None:
                self._layers.append(LayerCache())
            elif kinds[i].paged:
                g = self.groups[layer_group[i]]
                self._layers.append(g.kind.layer_cache(g.storage, g.layers.index(i), layer_group[i]))
            else:
                st = kinds[i].allocate_state(spec, max_requests, device) if device is not None else None
                self._layers.append(LayerCache(-1, True, None, None, st))
                self._state_layers.append(i)
                self._state_kinds[i] = kinds[i]
        for i, j in enumerate(cache_of):
            if j is not None:
                src = self._layers[j]
                self._layers[i] = LayerCache(src.group, False, src.k_pool, src.v_pool, src.state, src.pages)

    def __del__(self):
        book = getattr(self, "_book", None)
        if book:
            self._lib.vxh_cache_destroy(book)
            self._book = None

    def _handle(self, request_id, create: bool = True) -> Optional[int]:
        if isinstance(request_id, int) and not isinstance(request_id, bool) and 0 <= request_id < (1 << 62):
            return request_id
        h = self._handles.get(request_id)
        if h is None and create:
            h = self._handles[request_id] = self._next_handle
            self._names[h] = request_id
            self._next_handle -= 1
        return h

    def _known(self, request_id) -> int:
        h = self._handle(request_id, create=False)
        if h is None:
            raise KeyError(request_id)
        return h

    def handles(self, request_ids) -> "ctypes.Array":
        """The library's ids of requests that hold cache, as a C array."""
        return native.int64_array(self._known(r) for r in request_ids)

    def zero_state(self, slot: int) -> None:
        for i in self._state_layers:
            st = self._layers[i].state
            if st is not None:
                self._state_kinds[i].clear_slot(st, slot)

    # -- what layers see -------------------------------------------------------
    def layer(self, i: int) -> LayerCache:
        return self._layers[i]

    # -- requests ---------------------------------------------------------------
    def add_request(self, request_id) -> Optional[int]:
        """Gives the request a state slot (zeroed) and empty block tables; None
        if no slot is free."""
        slot = self._lib.vxh_cache_add(self._book, self._handle(request_id))
        if slot == -1:
            return None
        if slot < 0:
            if slot == native.ERR_ACCOUNTING:
                raise CacheAccountingError("request %r already holds cache" % (request_id,))
            native.check(slot)
        self.zero_state(slot)
        return slot

    def has_request(self, request_id) -> bool:
        h = self._handle(request_id, create=False)
        return h is not None and bool(self._lib.vxh_cache_has(self._book, h))

    def length(self, request_id) -> int:
        return int(native.check(self._lib.vxh_cache_length(self._book, self._known(request_id))))

    def pages_needed(self, request_id, new_tokens: int) -> List[int]:
        """Per group, the pages `reserve` would have to take for `new_tokens` more positions."""
        out = (ctypes.c_int * max(len(self.groups), 1))()
        native.check(self._lib.vxh_cache_pages_needed(self._book, self._known(request_id), int(new_tokens), out))
        return list(out[:len(self.groups)])

    def can_reserve(self, request_id, new_tokens: int) -> bool:
        return bool(native.check(self._lib.vxh_cache_can_reserve(self._book, self._known(request_id), int(new_tokens))))

    def reserve(self, request_id, new_tokens: int) -> bool:
        """Takes, in every group, the pages for positions [length, length + new_tokens);
        all or nothing.  False if some group has too few free pages."""
        return bool(native.check(self._lib.vxh_cache_reserve(self._book, self._known(request_id), int(new_tokens))))

    def commit(self, request_id, new_tokens: int) -> None:
        """The step has written `new_tokens` positions: advance, and give back
        pages that every later query's window has passed."""
        native.check(self._lib.vxh_cache_commit(self._book, self._known(request_id), int(new_tokens)))

    def release(self, request_id) -> None:
        """Gives back everything the request holds."""
        h = self._known(request_id)
        native.check(self._lib.vxh_cache_release(self._book, h))
        if h < 0:
            del self._handles[request_id]
            del self._names[h]

    # -- accounting ---------------------------------------------------------------
    def free_pages(self) -> List[int]:
        return [g.allocator.num_free for g in self.groups]

    def check(self) -> None:
        """Every page is either free or held by exactly as many tables as its
        count says; raises otherwise."""
        native.check(self._lib.vxh_cache_check(self._book))
