"""Cache manager: paged keys/values per cache group, block tables, state slots."""
from .manager import CacheGroup, CacheManager, PagedCacheView, RequestCache, StateCacheView
from .pools import OutOfPages, OutOfSlots, PagePool, StateSlotPool

__all__ = ["CacheGroup", "CacheManager", "PagedCacheView", "RequestCache", "StateCacheView",
           "OutOfPages", "OutOfSlots", "PagePool", "StateSlotPool"]
