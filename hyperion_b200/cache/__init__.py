from .manager import NO_PAGE, CacheError, CacheManager, OutOfPages, PagePool

__all__ = ["NO_PAGE", "CacheError", "CacheManager", "OutOfPages", "PagePool"]
