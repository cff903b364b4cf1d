from .manager import CacheGroup, CacheManager, OutOfSlots
from .page_pool import OutOfPages, PagePool

__all__ = ["CacheGroup", "CacheManager", "OutOfPages", "OutOfSlots", "PagePool"]
