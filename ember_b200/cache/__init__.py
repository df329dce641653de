"""Paged key/value cache: host-side manager and device storage."""
from .manager import CacheError, CacheGroup, CacheManager, PagePool, RequestCache, group_needs

__all__ = ["CacheError", "CacheGroup", "CacheManager", "PagePool", "RequestCache", "group_needs"]
