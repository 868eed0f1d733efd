from .manager import CacheError, CacheManager, OutOfPages, PagePool

__all__ = ["CacheError", "CacheManager", "OutOfPages", "PagePool"]
