"""The host side's native core (``runtime.cpp``) behind thin Python faces.

What is native: the cache's bookkeeping (pools of slots and pages, per-slot page lists, page-table
rows, lengths), the layout of a step's index arrays, the cutting of a long step into chunks, and the
generation loop's arithmetic (which requests start together, when a sequence ends).  What is not: the
tensors (torch owns device memory, streams and graphs), the composition of parts into a model and the
loops that call ``Model.step``.  The library is compiled by the C++ compiler the first time it is
used (no CUDA in it, so the tests that need no GPU exercise it), like the kernels' libraries.

Errors come back as codes with a message kept on the object (or per thread for the free functions);
they are raised here as :class:`CacheFull`, :class:`CacheError` or ``ValueError``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_void_p
from typing import Dict, List, Sequence, Tuple

import numpy as np

FULL, MISUSE, BAD_ARG = -1, -2, -3
_lib = None


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the tokens asked for."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        from ..csrc.build import load_library
        L = load_library("host_runtime")
        ll_p, int_p = POINTER(c_longlong), POINTER(c_int)
        sig = {
            "ssb_free_list_new": (c_void_p, [c_int, c_char_p]),
            "ssb_free_list_delete": (None, [c_void_p]),
            "ssb_free_list_error": (c_char_p, [c_void_p]),
            "ssb_free_list_take": (c_int, [c_void_p]),
            "ssb_free_list_give_back": (c_int, [c_void_p, c_int]),
            "ssb_free_list_n_free": (c_int, [c_void_p]),
            "ssb_free_list_is_held": (c_int, [c_void_p, c_int]),
            "ssb_free_list_check": (c_int, [c_void_p]),
            "ssb_cache_book_new": (c_void_p, [c_int, int_p, c_int, c_int, c_int, c_longlong]),
            "ssb_cache_book_delete": (None, [c_void_p]),
            "ssb_cache_book_error": (c_char_p, [c_void_p]),
            "ssb_cache_book_bind_table": (c_int, [c_void_p, c_int, c_void_p]),
            "ssb_cache_book_acquire": (c_int, [c_void_p]),
            "ssb_cache_book_release": (c_int, [c_void_p, c_int]),
            "ssb_cache_book_is_held": (c_int, [c_void_p, c_int]),
            "ssb_cache_book_length": (c_longlong, [c_void_p, c_int]),
            "ssb_cache_book_reserve": (c_int, [c_void_p, c_int, c_longlong]),
            "ssb_cache_book_advance": (c_int, [c_void_p, c_int, c_longlong]),
            "ssb_cache_book_reserve_each": (c_int, [c_void_p, c_int, int_p, c_longlong]),
            "ssb_cache_book_advance_each": (c_int, [c_void_p, c_int, int_p, c_longlong]),
            "ssb_cache_book_lengths": (c_int, [c_void_p, c_int, int_p, ll_p]),
            "ssb_cache_book_take_dirty": (c_int, [c_void_p, c_int, int_p, int_p]),
            "ssb_cache_book_free_slots": (c_int, [c_void_p]),
            "ssb_cache_book_free_pages": (c_int, [c_void_p, c_int]),
            "ssb_cache_book_held_pages": (c_int, [c_void_p, c_int]),
            "ssb_cache_book_pages_of": (c_int, [c_void_p, c_int, c_int, int_p, c_int]),
            "ssb_cache_book_check": (c_int, [c_void_p]),
            "ssb_decode_pages_bucket": (c_int, [c_longlong]),
            "ssb_host_error": (c_char_p, []),
            "ssb_pack_step": (c_int, [c_int, int_p, ll_p, ll_p, ll_p, ll_p, ll_p, c_longlong, c_void_p, c_longlong, ll_p]),
            "ssb_plan_chunks": (c_longlong, [c_int, ll_p, c_longlong, ll_p, c_longlong]),
            "ssb_plan_batch": (c_int, [c_int, ll_p, c_longlong, c_longlong, c_int, c_int, c_int]),
            "ssb_finished": (c_int, [c_longlong, c_longlong, c_longlong, ll_p, c_int]),
            "ssb_finished_rows": (c_int, [c_int, ll_p, ll_p, c_longlong, ll_p, c_int, int_p]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _raise(code: int, message: bytes):
    text = (message or b"").decode("utf-8", "replace")
    if code == FULL:
        raise CacheFull(text)
    if code == MISUSE:
        raise CacheError(text)
    raise ValueError(text)


def _ints(values) -> "ctypes.Array":
    values = list(values)
    return (c_int * max(len(values), 1))(*values)


def _longs(values) -> "ctypes.Array":
    values = list(values)
    return (c_longlong * max(len(values), 1))(*values)


class FreeList:
    """Ids 0..n-1, handed out lowest-first and taken back; freed ids are used again."""

    def __init__(self, n: int, what: str):
        if n <= 0:
            raise CacheError(f"a pool of {what}s needs at least one, got {n}")
        self._n = n
        self._h = c_void_p(lib().ssb_free_list_new(n, what.encode()))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.ssb_free_list_delete(h)

    def _ok(self, code: int) -> int:
        if code < 0:
            _raise(code, lib().ssb_free_list_error(self._h))
        return code

    @property
    def capacity(self) -> int:
        return self._n

    @property
    def n_free(self) -> int:
        return lib().ssb_free_list_n_free(self._h)

    @property
    def n_held(self) -> int:
        return self._n - self.n_free

    def is_held(self, i: int) -> bool:
        return bool(lib().ssb_free_list_is_held(self._h, int(i)))

    def take(self) -> int:
        return self._ok(lib().ssb_free_list_take(self._h))

    def take_many(self, n: int) -> List[int]:
        if n > self.n_free:
            raise CacheFull(f"{n} ids asked for, {self.n_free} of {self._n} are free")
        return [self.take() for _ in range(n)]

    def give_back(self, i: int) -> None:
        self._ok(lib().ssb_free_list_give_back(self._h, int(i)))

    def check(self) -> None:
        self._ok(lib().ssb_free_list_check(self._h))


class CacheBook:
    """Who holds which slot and which pages, for every group of cache entries: see ``runtime.cpp``.
    ``windows[g]`` is group g's window in tokens or None; ``tables[g]`` its page table on the host, an
    int32 array ``[max_slots, pages_per_seq]`` (for instance the numpy view of a pinned tensor) that the
    book writes the ids of reserved pages into."""

    def __init__(self, windows: Sequence, n_pages: int, pages_per_seq: int, max_slots: int, max_seq_tokens: int,
                 tables: Sequence[np.ndarray]):
        w = _ints([int(x) if x else 0 for x in windows])
        h = lib().ssb_cache_book_new(len(windows), w, n_pages, pages_per_seq, max_slots, max_seq_tokens)
        if not h:
            raise CacheError("the cache needs at least one page, one slot and room for one token")
        self._h = c_void_p(h)
        self.n_groups, self.max_slots = len(windows), max_slots
        self._tables = list(tables)                 # kept alive: the book writes into them
        for g, t in enumerate(self._tables):
            if t.dtype != np.int32 or t.shape != (max_slots, pages_per_seq) or not t.flags["C_CONTIGUOUS"]:
                raise CacheError("a page table must be a contiguous int32 array [slots, pages per sequence]")
            self._ok(lib().ssb_cache_book_bind_table(self._h, g, t.ctypes.data_as(c_void_p)))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.ssb_cache_book_delete(h)

    def _ok(self, code: int) -> int:
        if code < 0:
            _raise(code, lib().ssb_cache_book_error(self._h))
        return code

    def acquire(self) -> int:
        return self._ok(lib().ssb_cache_book_acquire(self._h))

    def release(self, slot: int) -> None:
        self._ok(lib().ssb_cache_book_release(self._h, int(slot)))

    def is_held(self, slot: int) -> bool:
        return bool(lib().ssb_cache_book_is_held(self._h, int(slot)))

    def length(self, slot: int) -> int:
        return self._ok(lib().ssb_cache_book_length(self._h, int(slot)))

    def lengths(self, slots: Sequence[int]) -> List[int]:
        out = (c_longlong * max(len(slots), 1))()
        self._ok(lib().ssb_cache_book_lengths(self._h, len(slots), _ints(slots), out))
        return list(out[:len(slots)])

    def reserve(self, slot: int, n_new: int) -> None:
        self._ok(lib().ssb_cache_book_reserve(self._h, int(slot), int(n_new)))

    def advance(self, slot: int, n_new: int) -> None:
        self._ok(lib().ssb_cache_book_advance(self._h, int(slot), int(n_new)))

    def reserve_each(self, slots: Sequence[int], n_new: int) -> None:
        self._ok(lib().ssb_cache_book_reserve_each(self._h, len(slots), _ints(slots), int(n_new)))

    def advance_each(self, slots: Sequence[int], n_new: int) -> None:
        self._ok(lib().ssb_cache_book_advance_each(self._h, len(slots), _ints(slots), int(n_new)))

    def take_dirty(self, group: int) -> Tuple[int, int]:
        """Rows ``[lo, hi)`` of the group's table that changed since the last call (empty: lo >= hi)."""
        lo, hi = c_int(), c_int()
        self._ok(lib().ssb_cache_book_take_dirty(self._h, group, ctypes.byref(lo), ctypes.byref(hi)))
        return lo.value, hi.value

    @property
    def free_slots(self) -> int:
        return lib().ssb_cache_book_free_slots(self._h)

    def free_pages(self, group: int) -> int:
        return lib().ssb_cache_book_free_pages(self._h, group)

    def held_pages(self, group: int) -> int:
        return lib().ssb_cache_book_held_pages(self._h, group)

    def pages_of(self, group: int, slot: int) -> Dict[int, int]:
        """Page index within the sequence -> page id, for the pages the slot holds now."""
        n = self._ok(lib().ssb_cache_book_pages_of(self._h, group, int(slot), (c_int * 2)(), 0))
        buf = (c_int * max(2 * n, 2))()
        self._ok(lib().ssb_cache_book_pages_of(self._h, group, int(slot), buf, n))
        return {buf[2 * i]: buf[2 * i + 1] for i in range(n)}

    def check(self) -> None:
        self._ok(lib().ssb_cache_book_check(self._h))


def decode_pages_bucket(longest: int) -> int:
    return lib().ssb_decode_pages_bucket(int(longest))


def pack_step(slots: Sequence[int], starts: Sequence[int], counts: Sequence[int], tokens: np.ndarray,
              want_counts: Sequence[int], want: Sequence[int], vocab_size) -> Tuple[np.ndarray, Tuple[int, ...]]:
    """The flat int32 array of a step (see ``ssb_pack_step``) and (T, B, W, max_new, max_total, is_decode)."""
    B = len(slots)
    T, W = int(sum(counts)), int(sum(want_counts))
    tokens = np.ascontiguousarray(tokens, dtype=np.int64)
    flat = np.empty(3 * T + 3 * B + 1 + W, dtype=np.int32)
    sizes = (c_longlong * 6)()
    rc = lib().ssb_pack_step(B, _ints(slots), _longs(starts), _longs(counts),
                             tokens.ctypes.data_as(POINTER(c_longlong)), _longs(want_counts), _longs(want),
                             int(vocab_size) if vocab_size else 0, flat.ctypes.data_as(c_void_p), flat.shape[0], sizes)
    if rc < 0:
        _raise(rc, lib().ssb_host_error())
    return flat, tuple(int(x) for x in sizes)


def plan_chunks(counts: Sequence[int], budget: int) -> List[List[tuple]]:
    """Cut a step of ``counts[i]`` tokens per entry into sub-steps of at most ``budget`` tokens: a list of
    chunks, a chunk a list of ``(entry, first, end)``."""
    cap = len(counts) + (int(sum(counts)) // max(int(budget), 1)) + 2
    out = (c_longlong * (4 * cap))()
    n = lib().ssb_plan_chunks(len(counts), _longs(counts), int(budget), out, cap)
    if n < 0:
        raise ValueError(lib().ssb_host_error().decode())
    chunks: List[List[tuple]] = []
    for i in range(n):
        c, e, lo, hi = out[4 * i:4 * i + 4]
        while len(chunks) <= c:
            chunks.append([])
        chunks[c].append((int(e), int(lo), int(hi)))
    return [c for c in chunks if c]


def plan_batch(prompt_lens_waiting: Sequence[int], max_new_tokens: int, free_tokens: int, free_slots: int,
               page_tokens: int, batch_size) -> int:
    """How many of the waiting requests (their prompt lengths, in arrival order) start together now."""
    return lib().ssb_plan_batch(len(prompt_lens_waiting), _longs(prompt_lens_waiting), int(max_new_tokens),
                                int(free_tokens), int(free_slots), int(page_tokens), int(batch_size or 0))


_WHY = {0: None, 1: "stop", 2: "length"}


def finished(token: int, n_generated: int, max_new_tokens: int, stop_ids) -> "str | None":
    stop = sorted(stop_ids)
    return _WHY[lib().ssb_finished(int(token), int(n_generated), int(max_new_tokens), _longs(stop), len(stop))]
