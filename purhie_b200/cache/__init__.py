"""Paged key/value cache with per-request block tables, layer groups and state slots."""
from .manager import CacheManager, CacheNeed, PageGroup, RequestCache
from .pages import OutOfPages, OutOfSlots, PageAllocator, SlotAllocator

__all__ = ["CacheManager", "CacheNeed", "PageGroup", "RequestCache", "OutOfPages", "OutOfSlots", "PageAllocator",
           "SlotAllocator"]
