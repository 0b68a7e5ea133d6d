"""Slots, paged keys and values, fixed-size per-sequence state."""
from .sequence_cache import (CacheError, FreeList, KVEntry, KVGroup, SequenceCache, StateEntry,  # noqa: F401
                             StateGroup, round_up)
