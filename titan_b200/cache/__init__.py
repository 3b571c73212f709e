from .cache import PAGE_SIZE, SequenceCache, SlotState
from .groups import CacheNeed, KVGroup, StateGroup
from .slots import CacheError, CacheFull, PagePool, SlotAllocator

__all__ = ["PAGE_SIZE", "SequenceCache", "SlotState", "CacheNeed", "KVGroup", "StateGroup", "CacheError",
           "CacheFull", "PagePool", "SlotAllocator"]
