from .manager import CacheGroup, CacheManager, KvNeed, RequestCache, StateNeed
from .pages import OutOfPages, PagePool

__all__ = ["CacheGroup", "CacheManager", "KvNeed", "OutOfPages", "PagePool", "RequestCache",
           "StateNeed"]
