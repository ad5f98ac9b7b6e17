"""Paged key/value cache, block tables, per-request state slots."""

from turingserve_b200.cache.allocator import NoFreePages, PageAllocator
from turingserve_b200.cache.manager import CacheManager, CacheView, RequestCache, RunNeeds

__all__ = ["NoFreePages", "PageAllocator", "CacheManager", "CacheView", "RequestCache", "RunNeeds"]
