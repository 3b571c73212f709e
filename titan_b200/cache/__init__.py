from .cache import PAGE_SIZE, SequenceCache, SlotState
from .groups import (CacheGeometry, CacheGroup, CacheNeed, KVGroup, StateGroup, build_cache_group,
                     register_cache_group)
from .slots import CacheError, CacheFull, PagePool, SlotAllocator

__all__ = ["PAGE_SIZE", "SequenceCache", "SlotState", "CacheNeed", "CacheGeometry", "CacheGroup", "KVGroup",
           "StateGroup", "register_cache_group", "build_cache_group", "CacheError", "CacheFull", "PagePool",
           "SlotAllocator"]
