from .manager import CacheGroup, CacheManager, LayerCache, OutOfPages, RequestCache
from .pages import CacheAccountingError, PageAllocator, SlotAllocator

__all__ = ["CacheGroup", "CacheManager", "LayerCache", "OutOfPages", "RequestCache", "CacheAccountingError",
           "PageAllocator", "SlotAllocator"]
