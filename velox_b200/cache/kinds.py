"""Kinds of cache: how what a mixer asks for (its `cache_spec()`) is stored.

The cache manager knows pages, block tables and slots; it does not know what lies
in a page.  For every kind of need, a `CacheKind` says
  * whether it is kept in pages (one entry per position, found through the
    request's block table) or in a slot (fixed size per request),
  * for pages: the window (0: every position stays), the bytes of one page of one
    layer, how the storage of a group of layers is allocated, and what a layer's
    mixer is handed (`LayerCache`),
  * for slots: the tensor [slots, ...] of one layer and how a slot is cleared.
A kind is registered for the class of its spec (`register_cache_kind`), from
anywhere: a test registers a cache of one latent vector per position without
touching this package.  Keys and values in pages (`PagedKV`) and fixed-size state
(`FixedState`) are registered here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..parts.base import FixedState, PagedKV


@dataclass
class LayerCache:
    """What a layer's mixer gets: its group (index into the step context's
    groups, -1 for none), whether it writes, and its storage: `k_pool`/`v_pool`
    for keys and values, `state` for a slot kind, `pages` for a paged kind with a
    layout of its own."""
    group: int = -1
    writes: bool = True
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    pages: Optional[torch.Tensor] = None


class CacheKind:
    paged = True

    # -- kinds kept in pages ---------------------------------------------------
    def window(self, spec) -> int:
        """Positions a query still reads (0: all).  Pages behind it are given back."""
        return 0

    def page_bytes(self, spec, page_size: int, element_bytes: int) -> int:
        """Bytes of one page of one layer."""
        raise NotImplementedError

    def allocate(self, spec, layers: int, num_pages: int, page_size: int, dtype, device) -> torch.Tensor:
        """Storage of a group of `layers` layers; its first dimension is the layer."""
        raise NotImplementedError

    def layer_cache(self, storage: Optional[torch.Tensor], index: int, group: int) -> LayerCache:
        """What layer `index` of the group's storage hands its mixer."""
        raise NotImplementedError

    # -- kinds kept in slots ---------------------------------------------------
    def allocate_state(self, spec, slots: int, device) -> torch.Tensor:
        raise NotImplementedError

    def clear_slot(self, state: torch.Tensor, slot: int) -> None:
        state[slot].zero_()


class PagedKVKind(CacheKind):
    """Keys and values of every position: [layer, K|V, page, kv head, offset in page,
    head_dim] (the reference keeps a K and a V pool [page, kv head, offset, head_dim]
    per layer, src/paged/pages.rs:62-74, 101-109)."""

    def window(self, spec: PagedKV) -> int:
        return spec.window

    def page_bytes(self, spec: PagedKV, page_size, element_bytes):
        return 2 * spec.num_kv_heads * spec.head_dim * page_size * element_bytes

    def allocate(self, spec: PagedKV, layers, num_pages, page_size, dtype, device):
        return torch.empty((layers, 2, num_pages, spec.num_kv_heads, page_size, spec.head_dim), dtype=dtype, device=device)

    def layer_cache(self, storage, index, group):
        if storage is None:
            return LayerCache(group, True)
        return LayerCache(group, True, storage[index, 0], storage[index, 1], None, storage[index])


class FixedStateKind(CacheKind):
    paged = False

    def allocate_state(self, spec: FixedState, slots, device):
        return torch.zeros((slots,) + tuple(spec.shape), dtype=getattr(torch, spec.dtype), device=device)


_KINDS: Dict[type, CacheKind] = {}


def register_cache_kind(spec_class: type, kind: CacheKind) -> CacheKind:
    _KINDS[spec_class] = kind
    return kind


def unregister_cache_kind(spec_class: type) -> None:
    _KINDS.pop(spec_class, None)


def cache_kind(spec) -> CacheKind:
    for cls in type(spec).__mro__:
        if cls in _KINDS:
            return _KINDS[cls]
    raise TypeError("a layer asks for a cache of unknown kind %r; registered kinds: %s"
                    % (spec, sorted(c.__name__ for c in _KINDS)))


register_cache_kind(PagedKV, PagedKVKind())
register_cache_kind(FixedState, FixedStateKind())
