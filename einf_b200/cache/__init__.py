"""The cache: page accounting (C++) and device storage."""
from .control import CacheManager, GroupSpec, PagePool
from .storage import CacheStorage

__all__ = ["CacheManager", "CacheStorage", "GroupSpec", "PagePool"]
