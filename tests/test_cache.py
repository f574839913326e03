"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from supersonic_b200.cache import (PAGE_TOKENS, CacheError, CacheFull, FreeList, KvNeed, SequenceCache,
                                   StateNeed, pages_for)


def make(max_tokens=64 * 8, max_seq=64 * 4, needs=None, **kw):
    needs = needs or {0: KvNeed(2, 16), 1: KvNeed(2, 16)}
    return SequenceCache(needs, max_tokens, max_seq, torch.float32, "cpu", **kw)


def test_free_list_is_strict():
    f = FreeList(3, "slot")
    a, b, c = f.take(), f.take(), f.take()
    assert (a, b, c) == (0, 1, 2) and f.n_free == 0
    with pytest.raises(CacheFull):
        f.take()
    f.give_back(b)
    with pytest.raises(CacheError, match="not held"):
        f.give_back(b)
    with pytest.raises(CacheError, match="does not exist"):
        f.give_back(7)
    assert f.take() == 1          # a freed id is used again
    f.check()


def test_slots_are_reused_and_lengths_reset():
    c = make()
    s0, s1 = c.acquire(), c.acquire()
    c.reserve(s0, 70); c.advance(s0, 70)
    assert c.length(s0) == 70 and c.kv_groups[0].pool.n_held == 2
    c.release(s0)
    with pytest.raises(CacheError, match="not held"):
        c.release(s0)
    with pytest.raises(CacheError, match="not held"):
        c.length(s0)
    again = c.acquire()
    assert again == s0 and c.length(again) == 0 and c.kv_groups[0].pool.n_held == 0
    c.check()
    c.release(again); c.release(s1)
    assert c.slots.n_free == c.max_slots and c.free_tokens() == 64 * 8


def test_pages_follow_lengths_and_tables_match():
    c = make()
    s = c.acquire()
    for n_new, want_pages in ((1, 1), (63, 1), (1, 2), (64, 3)):
        c.reserve(s, n_new); c.advance(s, n_new)
        g = c.kv_groups[0]
        assert len(g.held[s]) == want_pages == pages_for(c.length(s))
        c.sync()
        assert all(int(g.table[s, p]) == pid for p, pid in g.held[s].items())
    c.check()


def test_running_out_is_refused_without_damage():
    c = make(max_tokens=64 * 3, max_seq=64 * 3)
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 128); c.advance(a, 128)
    with pytest.raises(CacheFull, match="pages"):
        c.reserve(b, 65)                       # needs 2, only 1 free: nothing is taken
    assert c.kv_groups[0].pool.n_free == 1
    c.reserve(b, 64); c.advance(b, 64)
    with pytest.raises(CacheFull, match="exceed"):
        c.reserve(a, 65)                       # beyond what one sequence may hold
    c.check()


def test_groups_by_need_have_their_own_storage():
    needs = {0: KvNeed(2, 16), 1: KvNeed(2, 16, window=32), 2: KvNeed(2, 16), 3: StateNeed(5), 4: KvNeed(1, 32)}
    c = make(needs=needs)
    assert sorted(sorted(g.entries) for g in c.kv_groups) == [[0, 2], [1], [4]]
    k0, _, _, g0 = c.kv(0)
    k2, _, _, g2 = c.kv(2)
    k1, _, _, g1 = c.kv(1)
    assert g0 is g2 and g1 is not g0 and k0.data_ptr() != k2.data_ptr()
    assert tuple(k0.shape) == (8, 2, PAGE_TOKENS, 16) and tuple(c.kv(4)[0].shape) == (8, 1, PAGE_TOKENS, 32)
    assert tuple(c.state(3).shape) == (c.max_slots, 5)


def test_fixed_state_is_zeroed_on_acquire():
    c = make(needs={0: KvNeed(1, 16), 1: StateNeed(3)})
    s = c.acquire()
    c.state(1)[s] = torch.tensor([1.0, 2.0, 3.0])
    c.release(s)
    assert c.acquire() == s and c.state(1)[s].tolist() == [0.0, 0.0, 0.0]


def test_window_group_gives_pages_back():
    c = make(max_tokens=64 * 16, max_seq=64 * 16, needs={0: KvNeed(1, 16, window=70), 1: KvNeed(1, 16)})
    win = next(g for g in c.kv_groups if g.need.window)
    full = next(g for g in c.kv_groups if not g.need.window)
    s = c.acquire()
    c.reserve(s, 300); c.advance(s, 300)
    # a query at position >= 300 reads keys >= 231: pages 3.. stay, 0..2 are given back
    assert sorted(win.held[s]) == [3, 4] and sorted(full.held[s]) == [0, 1, 2, 3, 4]
    for _ in range(200):
        c.reserve(s, 1); c.advance(s, 1)
    assert min(win.held[s]) == (500 - 70 + 1) // 64 and len(win.held[s]) <= 3
    c.check()
    c.release(s)
    assert win.pool.n_held == 0 and full.pool.n_held == 0


def test_random_traffic_keeps_invariants():
    rnd = random.Random(0)
    c = make(max_tokens=64 * 12, max_seq=64 * 6, needs={0: KvNeed(1, 16), 1: KvNeed(1, 16, window=40)})
    live = []
    for _ in range(600):
        op = rnd.random()
        try:
            if op < 0.3:
                live.append(c.acquire())
            elif op < 0.8 and live:
                s = rnd.choice(live)
                n = rnd.choice([1, 1, 1, 17, 64, 100])
                c.reserve(s, n); c.advance(s, n)
            elif live:
                c.release(live.pop(rnd.randrange(len(live))))
        except CacheFull:
            pass
        c.check()
    for s in live:
        c.release(s)
    c.check()
    assert all(g.pool.n_held == 0 for g in c.kv_groups) and c.slots.n_held == 0


def test_generator_seed_is_never_zero():
    c = make()
    s = c.acquire(rng_seed=0)
    assert int(c.rng_state[s]) != 0
    c.seed(s, (1 << 64) - 1)
    assert int(c.rng_state[s]) == -1


def test_the_size_estimate_is_what_a_cache_allocates():
    """``bytes_needed`` (what the preflight compares with the device's free memory before anything
    is allocated) equals the bytes of the tensors a cache of those needs then holds."""
    needs = {0: KvNeed(2, 16), 1: KvNeed(2, 16, window=32), 2: KvNeed(2, 16), 3: StateNeed(5), 4: KvNeed(1, 32)}
    for dtype in (torch.float32, torch.bfloat16):
        for max_tokens, max_seq, slots in ((64 * 8, 64 * 4, None), (1000, 130, 3), (64, 4096, 7)):
            c = SequenceCache(needs, max_tokens, max_seq, dtype, "cpu", max_slots=slots)
            assert SequenceCache.bytes_needed(needs, max_tokens, max_seq, dtype, slots) == c.bytes_held()
    # Llama-3.1-8B sizes, 64 sequences of 8,192 tokens in bfloat16: 64 GiB of keys and values
    big = {i: KvNeed(8, 128) for i in range(32)}
    need = SequenceCache.bytes_needed(big, 64 * 8192, 8192, torch.bfloat16, 64)
    assert 64 * 2 ** 30 <= need < 64 * 2 ** 30 + 2 ** 20


def test_a_slot_opened_without_a_seed_starts_from_its_own_fixed_state():
    """Never zero (the fixed point of xorshift64), never what the slot's last sequence left."""
    import torch
    from supersonic_b200.cache import KvNeed, SequenceCache
    cache = SequenceCache({0: KvNeed(1, 16)}, 256, 128, torch.float32, "cpu", max_slots=3)
    a = cache.acquire()
    first = int(cache.rng_state[a])
    assert first != 0
    cache.rng_state[a] = 12345                  # a sequence drew from it
    cache.release(a)
    b = cache.acquire()
    assert b == a and int(cache.rng_state[b]) == first
    c = cache.acquire()
    assert int(cache.rng_state[c]) not in (0, first)
    d = cache.acquire(rng_seed=0)               # an explicit zero seed is replaced, as the reference does
    assert int(cache.rng_state[d]) != 0


def test_the_sequence_limit_is_the_one_asked_for_not_its_page_rounding():
    import pytest
    import torch
    from supersonic_b200.cache import CacheFull, KvNeed, SequenceCache
    cache = SequenceCache({0: KvNeed(1, 16)}, 512, 100, torch.float32, "cpu")
    assert cache.max_seq_tokens == 100
    s = cache.acquire()
    cache.reserve(s, 100)
    cache.advance(s, 100)
    with pytest.raises(CacheFull):
        cache.reserve(s, 1)
    cache.check()
