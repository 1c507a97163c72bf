from .manager import CacheGroup, CacheManager, LayerCache, PagedKeyValues, PagedNeed, PagedRows, RequestState
from .pages import PageCapacityError, PagePool

__all__ = ["CacheGroup", "CacheManager", "LayerCache", "PagedKeyValues", "PagedNeed", "PagedRows", "RequestState",
           "PageCapacityError", "PagePool"]
