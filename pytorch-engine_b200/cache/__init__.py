"""The paged cache: slots, pages, groups of layers with storage of their own, fixed-size state."""
from .pages import CacheBookkeepingError, CacheFull, NumberPool
from .paged import PAGE_TOKENS, CacheGroup, CacheView, PagedCache, pages_for

__all__ = ["CacheBookkeepingError", "CacheFull", "NumberPool", "PAGE_TOKENS", "CacheGroup", "CacheView",
           "PagedCache", "pages_for"]
