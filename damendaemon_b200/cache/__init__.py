from .manager import CacheGroup, CacheManager, LayerCache, PagedKeyValues, PagedNeed, RequestState
from .pages import PageCapacityError, PagePool

__all__ = ["CacheGroup", "CacheManager", "LayerCache", "PagedKeyValues", "PagedNeed", "RequestState",
           "PageCapacityError", "PagePool"]
