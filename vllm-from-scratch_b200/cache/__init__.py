"""Pages, block tables and state slots."""

from .manager import RELEASED, CacheError, CacheManager
from .pool import PagePool, PagePoolError
from .storage import CacheGroup, CacheStorage

__all__ = ["RELEASED", "CacheError", "CacheGroup", "CacheManager", "CacheStorage", "PagePool",
           "PagePoolError"]
