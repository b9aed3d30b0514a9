from .manager import CacheError, CacheGroup, CacheManager, IdPool, OutOfPages, RequestCache

__all__ = ["CacheError", "CacheGroup", "CacheManager", "IdPool", "OutOfPages", "RequestCache"]
