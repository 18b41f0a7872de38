"""The cache: slots, pages, groups of layers with their own storage, per-sequence state."""
from .allocator import Pool, PoolError
from .sequence_cache import PAGE, CacheError, CacheGroup, CacheView, SequenceCache

__all__ = ["PAGE", "CacheError", "CacheGroup", "CacheView", "Pool", "PoolError", "SequenceCache"]
