from .manager import CacheGroup, CacheGroupSpec, CacheManager, RequestCache, StateSlots, StateSpec
from .pages import OutOfPages, PagePool

__all__ = ["CacheGroup", "CacheGroupSpec", "CacheManager", "RequestCache", "StateSlots", "StateSpec", "OutOfPages",
           "PagePool"]
