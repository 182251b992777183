from kairyu_b200.cache.manager import CacheGroup, CacheLayout, CacheManager, RequestCache, StateBinding
from kairyu_b200.cache.page_pool import OutOfPages, PagePool
from kairyu_b200.cache.storage import CacheStorage

__all__ = [
    "CacheGroup", "CacheLayout", "CacheManager", "CacheStorage", "OutOfPages", "PagePool", "RequestCache", "StateBinding",
]
