from .needs import CacheBundle, FixedState, PagedKV
from .pages import OutOfPages, PagePool
from .manager import CacheManager, CacheView

__all__ = ["CacheBundle", "FixedState", "PagedKV", "OutOfPages", "PagePool", "CacheManager", "CacheView"]
