from .manager import CacheError, CacheManager, PageGroup
from .pages import BlockTable, OutOfPages, PageAllocator, PageError

__all__ = ["CacheError", "CacheManager", "PageGroup", "BlockTable", "OutOfPages", "PageAllocator", "PageError"]
