from .manager import CacheError, CacheManager, GroupSpec, OutOfPages

__all__ = ["CacheError", "CacheManager", "GroupSpec", "OutOfPages"]
