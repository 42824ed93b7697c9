from .pages import CacheCapacityError, CacheRollbackError, CacheStateError, FreeList
from .requests import PagedKVRequest, PagedLatentRequest, StateRequest
from .cache import PAGE, Cache, LatentView, PagedGroup, PagedView, StateGroup, pages_for

__all__ = ["CacheCapacityError", "CacheRollbackError", "CacheStateError", "FreeList", "PagedKVRequest",
           "PagedLatentRequest", "StateRequest", "PAGE", "Cache", "LatentView", "PagedGroup", "PagedView",
           "StateGroup", "pages_for"]
