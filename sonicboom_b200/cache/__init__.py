"""The paged key/value cache, its slot table and per-sequence state."""
from .kv import PAGE_SIZE, Cache, CacheGroup, KVNeed, SlotRecord, StateNeed
from .pages import CacheError, CacheFull, FreeList

__all__ = ["PAGE_SIZE", "Cache", "CacheGroup", "KVNeed", "SlotRecord", "StateNeed", "CacheError",
           "CacheFull", "FreeList"]
