"""The cache manager: pages of keys and values with a block table per request,
in groups of layers with the same needs, and slots for fixed-size state.

The manager is told, for every place of the model's running order, what the
mixer there needs (a layer that runs twice has two places and two caches).
Places that ask for the same `PagedKV` (kv heads, head size, window) form a
group.  A group has its own page pool, storage
[layer, K|V, page, kv head, offset in page, head_dim] (the reference keeps a K
and a V pool [page, kv head, offset, head_dim] per layer,
src/paged/pages.rs:62-74, 101-109), and its own block table per request: entry i
is the page that holds positions [i*S, (i+1)*S), or -1.  Pages are taken when a
step needs them (`reserve`), not for the worst case at admission as the
reference does (src/paged/scheduler.rs:255).  They are given back when the
request ends, and in a group with a window as soon as every position of a page
lies before the window of the next query; the freed page is the next one handed
out.

Layers whose mixers ask for `FixedState` get one tensor [slots, *shape] each;
a request holds one slot id from admission to its end, in every such layer.
Qwen3 has no such layer; the slot is assigned all the same.

The bookkeeping is host-only and runs without a device (`device=None`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import FixedState, PagedKV
from .pages import CacheAccountingError, PageAllocator, SlotAllocator


@dataclass
class LayerCache:
    """What a layer's mixer gets: its group (index into the step context's
    groups, -1 for none), whether it writes, and its storage."""
    group: int = -1
    writes: bool = True
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None


@dataclass
class CacheGroup:
    spec: PagedKV
    layers: List[int]
    allocator: PageAllocator
    storage: Optional[torch.Tensor] = None  # [layers, 2, pages, Hk, S, D]

    @property
    def window(self) -> int:
        return self.spec.window


@dataclass
class RequestCache:
    slot: int
    length: int = 0  # positions whose keys/values (or state) are in the cache
    tables: List[List[int]] = field(default_factory=list)  # per group


class OutOfPages(RuntimeError):
    pass


class CacheManager:
    def __init__(self, cache_specs: Sequence, cache_of: Sequence[Optional[int]], page_size: int, num_pages: int,
                 max_requests: int, max_blocks: int, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None, poison: bool = False):
        self.page_size, self.max_blocks = int(page_size), int(max_blocks)
        self.dtype, self.device = dtype, device
        self.groups: List[CacheGroup] = []
        self.slots = SlotAllocator(max_requests)
        self.requests: Dict[object, RequestCache] = {}
        # Host mirrors for building a step's description without loops: per group the
        # block table of every slot (-1 where no page is held), and every slot's length.
        self.table_of_slot: List[np.ndarray] = []
        self.length_of_slot = np.zeros(max_requests, np.int64)
        self._layers: List[LayerCache] = []
        self._state_layers: List[int] = []
        by_spec: Dict[PagedKV, int] = {}
        n_layers = len(cache_specs)
        layer_group = [-1] * n_layers
        for i, spec in enumerate(cache_specs):
            if isinstance(spec, PagedKV):
                if spec not in by_spec:
                    by_spec[spec] = len(self.groups)
                    self.groups.append(CacheGroup(spec, [], PageAllocator(num_pages)))
                layer_group[i] = by_spec[spec]
                self.groups[by_spec[spec]].layers.append(i)
        self.table_of_slot = [np.full((max_requests, self.max_blocks), -1, np.int32) for _ in self.groups]
        for g in self.groups:
            if device is not None:
                shape = (len(g.layers), 2, num_pages, g.spec.num_kv_heads, self.page_size, g.spec.head_dim)
                g.storage = torch.empty(shape, dtype=dtype, device=device)
                if poison:
                    g.storage.fill_(float("nan"))
                else:
                    g.storage.zero_()
        for i, spec in enumerate(cache_specs):
            if isinstance(spec, PagedKV):
                g = self.groups[layer_group[i]]
                j = g.layers.index(i)
                k = g.storage[j, 0] if g.storage is not None else None
                v = g.storage[j, 1] if g.storage is not None else None
                self._layers.append(LayerCache(layer_group[i], True, k, v, None))
            elif isinstance(spec, FixedState):
                st = None
                if device is not None:
                    st = torch.zeros((max_requests,) + tuple(spec.shape), dtype=getattr(torch, spec.dtype), device=device)
                self._layers.append(LayerCache(-1, True, None, None, st))
                self._state_layers.append(i)
            elif spec is None:
                self._layers.append(LayerCache())
            else:
                raise TypeError("layer %d asks for a cache of unknown kind %r" % (i, spec))
        for i, j in enumerate(cache_of):
            if j is not None:
                src = self._layers[j]
                self._layers[i] = LayerCache(src.group, False, src.k_pool, src.v_pool, src.state)

    # -- what layers see -------------------------------------------------------
    def layer(self, i: int) -> LayerCache:
        return self._layers[i]

    # -- requests ---------------------------------------------------------------
    def add_request(self, request_id) -> Optional[int]:
        """Gives the request a state slot (zeroed) and empty block tables; None
        if no slot is free."""
        if request_id in self.requests:
            raise CacheAccountingError("request %r already holds cache" % (request_id,))
        slot = self.slots.alloc()
        if slot is None:
            return None
        self.requests[request_id] = RequestCache(slot, 0, [[] for _ in self.groups])
        self.length_of_slot[slot] = 0
        for t in self.table_of_slot:
            t[slot, :] = -1
        for i in self._state_layers:
            st = self._layers[i].state
            if st is not None:
                st[slot].zero_()
        return slot

    def has_request(self, request_id) -> bool:
        return request_id in self.requests

    def length(self, request_id) -> int:
        return self.requests[request_id].length

    def _first_needed_page(self, g: CacheGroup, next_position: int) -> int:
        """Index of the first page that the query at `next_position` can still see."""
        if g.window <= 0:
            return 0
        first_key = max(0, next_position + 1 - g.window)
        return first_key // self.page_size

    def pages_needed(self, request_id, new_tokens: int) -> List[int]:
        """Per group, the pages `reserve` would have to take for `new_tokens` more positions."""
        rc = self.requests[request_id]
        want = -(-(rc.length + new_tokens) // self.page_size)
        return [max(0, want - len(t)) for t in rc.tables]

    def can_reserve(self, request_id, new_tokens: int) -> bool:
        need = self.pages_needed(request_id, new_tokens)
        return all(n <= g.allocator.num_free for n, g in zip(need, self.groups))

    def reserve(self, request_id, new_tokens: int) -> bool:
        """Takes, in every group, the pages for positions [length, length + new_tokens);
        all or nothing.  False if some group has too few free pages."""
        rc = self.requests[request_id]
        if rc.length + new_tokens > self.max_blocks * self.page_size:
            raise OutOfPages("request %r would reach %d positions; block tables hold %d"
                             % (request_id, rc.length + new_tokens, self.max_blocks * self.page_size))
        need = self.pages_needed(request_id, new_tokens)
        if any(n > g.allocator.num_free for n, g in zip(need, self.groups)):
            return False
        for n, g, table, mirror in zip(need, self.groups, rc.tables, self.table_of_slot):
            if n:
                pages = g.allocator.alloc(n)
                mirror[rc.slot, len(table):len(table) + n] = pages
                table.extend(pages)
        return True

    def commit(self, request_id, new_tokens: int) -> None:
        """The step has written `new_tokens` positions: advance, and give back
        pages that every later query's window has passed."""
        rc = self.requests[request_id]
        rc.length += new_tokens
        self.length_of_slot[rc.slot] = rc.length
        for g, table, mirror in zip(self.groups, rc.tables, self.table_of_slot):
            if len(table) * self.page_size < rc.length:
                raise CacheAccountingError("request %r wrote %d positions into %d pages"
                                           % (request_id, rc.length, len(table)))
            if g.window > 0:
                keep_from = self._first_needed_page(g, rc.length)
                for i in range(min(keep_from, len(table))):
                    if table[i] >= 0:
                        g.allocator.free([table[i]])
                        table[i] = -1
                        mirror[rc.slot, i] = -1

    def release(self, request_id) -> None:
        """Gives back everything the request holds."""
        rc = self.requests.pop(request_id)
        for g, table in zip(self.groups, rc.tables):
            g.allocator.free([p for p in table if p >= 0])
        self.slots.free(rc.slot)

    # -- accounting ---------------------------------------------------------------
    def free_pages(self) -> List[int]:
        return [g.allocator.num_free for g in self.groups]

    def check(self) -> None:
        """Every page is either free or held by exactly as many tables as its
        count says; raises otherwise."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, int] = {}
            for rc in self.requests.values():
                for p in rc.tables[gi]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            free = set(g.allocator._free)
            if len(free) != len(g.allocator._free):
                raise CacheAccountingError("group %d: a page is on the free list twice" % gi)
            for p in range(g.allocator.num_pages):
                rcnt = g.allocator.refcount(p)
                if (p in free) != (rcnt == 0) or held.get(p, 0) != rcnt:
                    raise CacheAccountingError(
                        "group %d page %d: count %d, held by %d tables, %s the free list"
                        % (gi, p, rcnt, held.get(p, 0), "on" if p in free else "not on"))
