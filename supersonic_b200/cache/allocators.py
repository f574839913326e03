"""Host-side bookkeeping of the cache: which slots and which pages are held.

The pools themselves are native (``supersonic_b200/host/runtime.cpp``); this module names them for
the cache.  No tensors: it can be tested without a GPU.  Every misuse (double free, freeing what was
never held, running out) raises :class:`CacheError` instead of corrupting state.  The reference has
no such pool: each sequence owns buffers that grow by reallocation in 256-token chunks
(crates/qwen35/src/state.rs:225-311).
"""
from __future__ import annotations

from ..host import CacheError, CacheFull, FreeList

__all__ = ["CacheError", "CacheFull", "FreeList"]
