from .manager import CacheManager, CacheView, PageAllocator, RequestCache
from .needs import PagedKVNeed, StateNeed

__all__ = ["CacheManager", "CacheView", "PageAllocator", "RequestCache", "PagedKVNeed", "StateNeed"]
