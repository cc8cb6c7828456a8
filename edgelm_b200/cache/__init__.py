from .cache import PAGE, CacheEntry, CompositeEntry, KVGroup, SequenceCache, StateGroup, pages_for
from .slots import CacheError, FreeList

__all__ = ["PAGE", "CacheEntry", "CompositeEntry", "KVGroup", "SequenceCache", "StateGroup", "pages_for", "CacheError", "FreeList"]
