from .manager import CacheGroup, CacheManager, LayerCache, PagedKeyValues, RequestState
from .pages import PageCapacityError, PagePool

__all__ = ["CacheGroup", "CacheManager", "LayerCache", "PagedKeyValues", "RequestState",
           "PageCapacityError", "PagePool"]
