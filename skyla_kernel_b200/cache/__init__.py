"""The sequence cache: slots, paged keys/values per layer group, per-slot state."""
from .kv import PAGE_SIZE, KVGroup, KVNeed, SequenceCache, StateNeed
from .slots import CacheError, CacheFull, FreeList

__all__ = ["PAGE_SIZE", "KVGroup", "KVNeed", "SequenceCache", "StateNeed", "CacheError",
           "CacheFull", "FreeList"]
