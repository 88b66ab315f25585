"""The cache manager: paged keys and values, block tables, state slots."""
from .manager import CacheError, CacheGroup, CacheManager, FreeList, OutOfPages, OutOfSlots, RequestCache
from .sizing import group_layout, pages_per_group

__all__ = ["CacheError", "CacheGroup", "CacheManager", "FreeList", "OutOfPages", "OutOfSlots", "RequestCache",
           "group_layout", "pages_per_group"]
