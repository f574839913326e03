"""Slots, paged keys and values, and fixed-size per-sequence state."""
from .allocators import CacheError, CacheFull, FreeList
from .sequence_cache import (PAGE_SHIFT, PAGE_TOKENS, KvGroup, KvNeed, SequenceCache,
                             StateNeed, pages_for)

__all__ = ["CacheError", "CacheFull", "FreeList", "PAGE_SHIFT", "PAGE_TOKENS", "KvGroup",
           "KvNeed", "SequenceCache", "StateNeed", "pages_for"]
