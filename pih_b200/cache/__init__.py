"""Cache manager: paged keys/values per cache group, block tables, state slots."""
# Tokens of a page unless the caller says otherwise.  A prompt's attention fetches a page of one head's keys with one
# TMA box; the copy engine spends about the same time on a box whatever its size, and with 16-token pages (2 KB a
# box, 32 boxes a 128-key tile) that time, not the arithmetic, bounded the kernel.  64 tokens is also the most that
# the tile of a box can hold.
DEFAULT_PAGE_SIZE = 64

from .manager import CacheGroup, CacheManager, PagedCacheView, RequestCache, StateCacheView
from .pools import OutOfPages, OutOfSlots, PagePool, StateSlotPool

__all__ = ["DEFAULT_PAGE_SIZE", "CacheGroup", "CacheManager", "PagedCacheView", "RequestCache", "StateCacheView",
           "OutOfPages", "OutOfSlots", "PagePool", "StateSlotPool"]
