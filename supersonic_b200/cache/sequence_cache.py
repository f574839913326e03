"""The cache: a slot per live sequence, keys and values per cache entry in pages,
fixed-size per-sequence state beside them.

Layout.  Mixers state what they need (:class:`KvNeed`: kv heads, head size,
window; :class:`StateNeed`: a number of float32 values).  Cache entries with the same need form a group
with storage of its own: ``k`` and ``v`` of shape ``[entries, pages, kv_heads,
PAGE_TOKENS, head_dim]`` and a page table ``[slots, pages_per_sequence]``.  A
sequence's tokens ``64p .. 64p+63`` of one kv head are contiguous, so a decode
block streams them and a bulk copy can fetch them.  A group with a window gives
pages back as soon as every later query is past them.

Per sequence the cache also keeps: its length (host), the state of its random
generator (device), and for every :class:`StateNeed` entry a zeroed float32
row (device).  The reference keeps ``kv_filled`` in ``LayerState`` and
fixed-size conv/recurrent buffers for its other layer kind
(crates/qwen35/src/state.rs:17-80, 314).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple, Union

import torch

from ..host import CacheBook
from .allocators import CacheError

PAGE_SHIFT = 6
PAGE_TOKENS = 1 << PAGE_SHIFT


@dataclass(frozen=True)
class KvNeed:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None       # None: every earlier key stays


@dataclass(frozen=True)
class StateNeed:
    n_values: int                      # float32 values per sequence


Need = Union[KvNeed, StateNeed]


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_TOKENS - 1) >> PAGE_SHIFT


class _Pool:
    """The page pool of one group as the bookkeeping sees it."""

    def __init__(self, book: CacheBook, group: int, capacity: int):
        self._book, self._group, self.capacity = book, group, capacity

    @property
    def n_free(self) -> int:
        return self._book.free_pages(self._group)

    @property
    def n_held(self) -> int:
        return self._book.held_pages(self._group)


class _HeldPages:
    """``held[slot]``: page index within the sequence -> page id, for the pages the slot holds now."""

    def __init__(self, book: CacheBook, group: int):
        self._book, self._group = book, group

    def __getitem__(self, slot: int) -> Dict[int, int]:
        return self._book.pages_of(self._group, slot)


class _Slots:
    """The slot pool as the bookkeeping sees it."""

    def __init__(self, book: CacheBook, capacity: int):
        self._book, self.capacity = book, capacity

    @property
    def n_free(self) -> int:
        return self._book.free_slots

    @property
    def n_held(self) -> int:
        return self.capacity - self._book.free_slots

    def is_held(self, slot: int) -> bool:
        return self._book.is_held(slot)


class KvGroup:
    """Storage of the cache entries that share one need.  Which pages a slot holds is kept by the
    cache's native book, which writes the page ids into ``table_host``; ``pool`` and ``held`` show it."""

    def __init__(self, need: KvNeed, entries: List[int], n_pages: int, max_slots: int,
                 pages_per_seq: int, dtype: torch.dtype, device: torch.device):
        self.need = need
        self.entries = list(entries)
        self.index_of = {e: i for i, e in enumerate(self.entries)}
        self.n_pages = n_pages
        self.pages_per_seq = pages_per_seq
        shape = (len(entries), n_pages, need.n_kv_heads, PAGE_TOKENS, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        pin = device.type == "cuda"
        self.table_host = torch.zeros((max_slots, pages_per_seq), dtype=torch.int32, pin_memory=pin)
        self.table = torch.zeros((max_slots, pages_per_seq), dtype=torch.int32, device=device)
        self.pool: Optional[_Pool] = None          # set by the cache once its book exists
        self.held: Optional[_HeldPages] = None
        self._book: Optional[CacheBook] = None
        self._index = -1

    def bind(self, book: CacheBook, index: int) -> None:
        self._book, self._index = book, index
        self.pool = _Pool(book, index, self.n_pages)
        self.held = _HeldPages(book, index)

    def sync(self) -> None:
        lo, hi = self._book.take_dirty(self._index)
        if hi > lo:
            self.table[lo:hi].copy_(self.table_host[lo:hi], non_blocking=True)


def default_seed(slot: int) -> int:
    """Generator state of a sequence opened without a seed: the reference's default sampling seed
    (42, crates/runner/src/main.rs:383) spread over the slots."""
    return (42 * 0x9E3779B97F4A7C15 + (slot + 1) * 0xD1342543DE82EF95) & ((1 << 64) - 1)


class SequenceCache:
    """Slots, page groups and per-sequence state for one model.

    ``needs`` maps a cache id (as named by the model's schedule) to what its mixer
    needs.  ``max_tokens`` bounds the tokens all live sequences hold together
    (each rounded up to whole pages); ``max_seq_tokens`` bounds one sequence.
    """

    def __init__(self, needs: Dict[int, Need], max_tokens: int, max_seq_tokens: int,
                 dtype: torch.dtype, device, max_slots: Optional[int] = None):
        device = torch.device(device)
        if max_tokens <= 0 or max_seq_tokens <= 0:
            raise CacheError("the cache needs room for at least one token")
        self.device, self.dtype = device, dtype
        self.n_pages = pages_for(max_tokens)
        self.pages_per_seq = min(pages_for(max_seq_tokens), self.n_pages)
        # the limit a sequence may reach is the one asked for, not its page-rounded figure: position
        # tables and other per-position data of the parts are sized by it
        self.max_seq_tokens = min(int(max_seq_tokens), self.pages_per_seq * PAGE_TOKENS)
        self.max_slots = max_slots if max_slots is not None else min(self.n_pages, 4096)
        self._preflight(needs, max_tokens, max_seq_tokens)
        # groups by need
        by_need: Dict[KvNeed, List[int]] = {}
        state_entries: List[Tuple[int, StateNeed]] = []
        for cid, need in sorted(needs.items()):
            if isinstance(need, KvNeed):
                by_need.setdefault(need, []).append(cid)
            elif isinstance(need, StateNeed):
                state_entries.append((cid, need))
            elif need is not None:
                raise CacheError(f"cache entry {cid}: unknown need {need!r}")
        self.kv_groups: List[KvGroup] = [
            KvGroup(need, entries, self.n_pages, self.max_slots, self.pages_per_seq, dtype, device)
            for need, entries in by_need.items()]
        # who holds which slot and page: the native book, which fills the groups' host page tables
        self._book = CacheBook([g.need.window for g in self.kv_groups], self.n_pages, self.pages_per_seq,
                               self.max_slots, self.max_seq_tokens, [g.table_host.numpy() for g in self.kv_groups])
        for i, g in enumerate(self.kv_groups):
            g.bind(self._book, i)
        self.slots = _Slots(self._book, self.max_slots)
        self._group_of: Dict[int, KvGroup] = {e: g for g in self.kv_groups for e in g.entries}
        self._state: Dict[int, torch.Tensor] = {
            cid: torch.zeros((self.max_slots, need.n_values), dtype=torch.float32, device=device)
            for cid, need in state_entries}
        self.rng_state = torch.zeros(self.max_slots, dtype=torch.int64, device=device)

    @staticmethod
    def bytes_needed(needs: Dict[int, Need], max_tokens: int, max_seq_tokens: int, dtype: torch.dtype,
                     max_slots: Optional[int] = None) -> int:
        """Device bytes a cache of these needs and sizes allocates: keys and values of every entry
        for every page, the page tables, fixed state and generator state of every slot."""
        n_pages = pages_for(max_tokens)
        pages_per_seq = min(pages_for(max_seq_tokens), n_pages)
        slots = max_slots if max_slots is not None else min(n_pages, 4096)
        item = torch.empty((), dtype=dtype).element_size()
        total = slots * 8                                                  # generator state
        seen = set()
        for need in needs.values():
            if isinstance(need, KvNeed):
                total += 2 * n_pages * need.n_kv_heads * PAGE_TOKENS * need.head_dim * item
                if need not in seen:                                       # one page table a group
                    seen.add(need)
                    total += slots * pages_per_seq * 4
            elif isinstance(need, StateNeed):
                total += slots * need.n_values * 4
        return total

    def _preflight(self, needs, max_tokens, max_seq_tokens) -> None:
        """Refuse a cache the device cannot hold before any of it is allocated (the reference
        checks a per-model memory budget before it loads: crates/runner/src/registry.rs:773-785)."""
        if self.device.type != "cuda":
            return
        need = self.bytes_needed(needs, max_tokens, max_seq_tokens, self.dtype, self.max_slots)
        free, total = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        if need > free:
            gib = 1 << 30
            raise CacheError(f"a cache of {max_tokens} tokens needs {need / gib:.1f} GiB; {free / gib:.1f} GiB of "
                             f"the device's {total / gib:.1f} GiB are free (the weights are loaded already): "
                             "ask for fewer tokens (context size x batch size, or max_tokens)")

    # ---- slots ------------------------------------------------------------------------
    def acquire(self, rng_seed: Optional[int] = None) -> int:
        """A free slot with length 0, zeroed fixed state and a seeded generator.  Without a seed
        the generator starts from a fixed state of the slot's own, never from zero (the fixed point
        of xorshift64) and never from what the slot's last sequence left."""
        slot = self._book.acquire()
        for t in self._state.values():
            t[slot].zero_()
        self.seed(slot, rng_seed if rng_seed is not None else default_seed(slot))
        return slot

    def seed(self, slot: int, seed: int) -> None:
        seed &= (1 << 64) - 1
        if seed == 0:
            seed = 0x9E3779B97F4A7C15       # xorshift needs a non-zero state (qwen36_moe_decode.rs:1091-1094)
        if seed >= 1 << 63:
            seed -= 1 << 64
        self.rng_state[slot] = seed

    def release(self, slot: int) -> None:
        """Give the slot and every page it holds back."""
        self._book.release(slot)

    def length(self, slot: int) -> int:
        return self._book.length(slot)

    def lengths(self, slots) -> List[int]:
        return self._book.lengths(list(slots))

    def live_slots(self) -> List[int]:
        return [s for s in range(self.max_slots) if self.slots.is_held(s)]

    # ---- per step -----------------------------------------------------------------------
    def reserve(self, slot: int, n_new: int) -> None:
        """Make room for ``n_new`` more tokens of ``slot`` in every group (all or nothing)."""
        self._book.reserve(slot, n_new)

    def advance(self, slot: int, n_new: int) -> None:
        """Record that ``n_new`` tokens were appended; window groups drop what nothing reads."""
        self._book.advance(slot, n_new)

    def reserve_each(self, slots, n_new: int = 1) -> None:
        """``reserve`` for every slot of a decode step, in one call."""
        self._book.reserve_each(list(slots), n_new)

    def advance_each(self, slots, n_new: int = 1) -> None:
        self._book.advance_each(list(slots), n_new)

    def sync(self) -> None:
        """Upload page-table rows that changed since the last call."""
        for g in self.kv_groups:
            g.sync()

    # ---- what parts read --------------------------------------------------------------
    def kv(self, cache_id: int):
        """(k, v, page_table, group) of one cache entry; k and v are ``[pages, kv_heads, 64, head_dim]``."""
        g = self._group_of[cache_id]
        i = g.index_of[cache_id]
        return g.k[i], g.v[i], g.table, g

    def state(self, cache_id: int) -> torch.Tensor:
        """Fixed-size state ``[slots, n_values]`` float32 of one cache entry."""
        return self._state[cache_id]

    def free_tokens(self) -> int:
        return min((g.pool.n_free for g in self.kv_groups), default=self.n_pages) * PAGE_TOKENS

    def bytes_read_for(self, slot: int) -> int:
        """Bytes of keys and values an attention over ``slot`` reads now: every cache entry, the
        tokens the sequence holds (a window group: at most its window), keys and values."""
        n = self.length(slot)
        total = 0
        for g in self.kv_groups:
            tokens = n if g.need.window is None else min(n, g.need.window)
            total += len(g.entries) * 2 * tokens * g.need.n_kv_heads * g.need.head_dim * g.k.element_size()
        return total + sum(t.shape[1] * 4 for t in self._state.values())

    def bytes_held(self) -> int:
        n = sum(g.k.numel() * g.k.element_size() * 2 + g.table.numel() * 4 for g in self.kv_groups)
        return n + sum(t.numel() * 4 for t in self._state.values()) + self.rng_state.numel() * 8

    def check(self) -> None:
        """Invariants: no slot or page lost or held twice; held pages match the tables."""
        self._book.check()
