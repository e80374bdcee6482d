from .kinds import CacheKind, cache_kind, register_cache_kind, unregister_cache_kind
from .manager import CacheGroup, CacheManager, LayerCache, OutOfPages, RequestCache
from .pages import CacheAccountingError, PageAllocator, SlotAllocator

__all__ = ["CacheGroup", "CacheKind", "CacheManager", "LayerCache", "OutOfPages", "RequestCache",
           "CacheAccountingError", "PageAllocator", "SlotAllocator", "cache_kind", "register_cache_kind",
           "unregister_cache_kind"]
