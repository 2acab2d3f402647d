from .manager import CacheGroup, CacheManager, KvNeed, RequestCache, StateNeed
from .pages import OutOfPages, PagePool
from .prefix import PrefixIndex, PrefixMatch

__all__ = ["CacheGroup", "CacheManager", "KvNeed", "OutOfPages", "PagePool", "PrefixIndex",
           "PrefixMatch", "RequestCache", "StateNeed"]
