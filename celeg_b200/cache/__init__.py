"""Cache manager: pages and block tables for growing caches, slots for fixed-size state."""
from .pages import OutOfPages, PageError, PagePool
from .manager import NO_PAGE, CacheManager, PagedGroup, PagedNeed, RequestCache, StateLayout, StateNeed

__all__ = ["OutOfPages", "PageError", "PagePool", "NO_PAGE", "CacheManager", "PagedGroup", "PagedNeed",
           "RequestCache", "StateLayout", "StateNeed"]
