"""The cache manager: paged keys and values, block tables, state slots."""
from .manager import CacheError, CacheGroup, CacheManager, FreeList, OutOfPages, OutOfSlots, RequestCache

__all__ = ["CacheError", "CacheGroup", "CacheManager", "FreeList", "OutOfPages", "OutOfSlots", "RequestCache"]
