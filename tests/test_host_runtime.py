"""The host side's native core (supersonic_b200/host/runtime.cpp) against plain Python restatements of
its rules: the layout of a step, the cutting of a long step, the choice of the next batch, the stop
rules, the page bucket, and the cache's book under random traffic."""
import random

import numpy as np
import pytest

from supersonic_b200 import host
from supersonic_b200.engine.batch import StepEntry, pack_entries


def plain_layout(entries, starts):
    tok, pos, slot_of, cu, want = [], [], [], [0], []
    for e, s in zip(entries, starts):
        base = cu[-1]
        want += [base + w for w in e.want]
        tok += list(e.tokens)
        pos += list(range(s, s + len(e.tokens)))
        slot_of += [e.slot] * len(e.tokens)
        cu.append(base + len(e.tokens))
    return tok + pos + slot_of + [e.slot for e in entries] + list(starts) + cu + want


def test_a_step_is_laid_out_as_the_kernels_read_it():
    rnd = random.Random(3)
    for _ in range(50):
        n = rnd.randint(1, 6)
        slots = rnd.sample(range(40), n)
        entries, starts = [], []
        for s in slots:
            t = rnd.choice([1, 1, 2, 7, 65])
            entries.append(StepEntry(s, [rnd.randrange(500) for _ in range(t)], sorted(rnd.sample(range(t), rnd.randint(0, min(t, 3))))))
            starts.append(rnd.choice([0, 3, 64, 1000]))
        p = pack_entries(entries, starts, vocab_size=500)
        assert p.flat.dtype == np.int32 and p.flat.tolist() == plain_layout(entries, starts)
        counts = [len(e.tokens) for e in entries]
        assert (p.n_tokens, p.n_seqs, p.n_want) == (sum(counts), n, sum(len(e.want) for e in entries))
        assert p.max_new == max(counts) and p.max_total == max(s + c for s, c in zip(starts, counts))
        assert p.slots == slots and p.starts == starts and p.counts == counts


def test_a_malformed_step_is_refused_with_its_reason():
    with pytest.raises(ValueError, match="at least one entry"):
        pack_entries([], [])
    with pytest.raises(ValueError, match="at least one token"):
        pack_entries([StepEntry(0, [], [])], [0])
    with pytest.raises(ValueError, match="wanted place 2 is outside its 2 tokens"):
        pack_entries([StepEntry(0, [1, 2], [2])], [0])
    with pytest.raises(ValueError, match="wanted place -1"):
        pack_entries([StepEntry(0, [1, 2], [-1])], [0])
    with pytest.raises(ValueError, match=r"token ids \[9, -4\] are outside the vocabulary of 9"):
        pack_entries([StepEntry(0, [1, 9], [0]), StepEntry(1, [-4], [0])], [0, 0], vocab_size=9)
    with pytest.raises(ValueError, match="slot appears twice"):
        pack_entries([StepEntry(3, [1], [0]), StepEntry(3, [2], [0])], [0, 0])
    pack_entries([StepEntry(0, [1, 900000], [0])], [0])                 # no vocabulary given: ids are not checked


def plain_chunks(counts, budget):
    chunks, room = [[]], budget
    for i, n in enumerate(counts):
        first = 0
        while first < n:
            if room == 0:
                chunks.append([])
                room = budget
            take = min(room, n - first)
            chunks[-1].append((i, first, first + take))
            first += take
            room -= take
    return [c for c in chunks if c]


def test_a_long_step_is_cut_into_chunks_within_the_budget():
    rnd = random.Random(5)
    for _ in range(200):
        counts = [rnd.choice([1, 2, 5, 64, 100, 333]) for _ in range(rnd.randint(1, 7))]
        budget = rnd.choice([1, 3, 64, 100, 1000])
        got = host.plan_chunks(counts, budget)
        assert got == plain_chunks(counts, budget)
        assert all(sum(hi - lo for _, lo, hi in c) <= budget for c in got)
        assert all(len({e for e, _, _ in c}) == len(c) for c in got)     # no entry twice in a chunk
    with pytest.raises(ValueError, match="at least 1"):
        host.plan_chunks([3], 0)


def plain_batch(lens, max_new, free_tokens, free_slots, page, batch_size):
    chosen, room = 0, free_tokens
    for n in lens:
        if chosen >= free_slots or (batch_size and chosen >= batch_size):
            break
        need = -(-(n + max(max_new, 1)) // page) * page
        if need > room:
            break
        chosen += 1
        room -= need
    return chosen


def test_the_next_batch_is_what_fits_in_arrival_order():
    rnd = random.Random(7)
    for _ in range(300):
        lens = [rnd.choice([1, 5, 63, 64, 65, 500]) for _ in range(rnd.randint(0, 9))]
        args = (rnd.choice([0, 1, 8, 200]), rnd.choice([0, 64, 640, 6400]), rnd.randint(0, 6), 64, rnd.choice([None, 0, 1, 3]))
        assert host.plan_batch(lens, *args) == plain_batch(lens, *args)


def test_a_sequence_ends_at_a_stop_token_or_at_its_budget():
    assert host.finished(5, 1, 8, {5, 9}) == "stop"
    assert host.finished(5, 8, 8, {5}) == "stop"                       # a stop token at the budget is a stop
    assert host.finished(4, 8, 8, {5}) == "length"
    assert host.finished(4, 7, 8, {5}) is None
    assert host.finished(4, 1, 0, ()) == "length"
    assert host.finished(4, 3, 8, frozenset()) is None


def test_the_page_bucket_is_the_largest_power_of_two_within_the_pages():
    for longest in list(range(0, 300)) + [4095, 4096, 4097, 131072, 10 ** 7]:
        pages = max(1, -(-longest // 64))
        assert host.decode_pages_bucket(longest) == 1 << (pages.bit_length() - 1)


def test_the_book_keeps_its_invariants_and_its_tables_under_random_traffic():
    rnd = random.Random(11)
    n_pages, per_seq, slots = 24, 8, 6
    tables = [np.zeros((slots, per_seq), dtype=np.int32) for _ in range(2)]
    book = host.CacheBook([None, 100], n_pages, per_seq, slots, per_seq * 64 - 7, tables)
    length = {}
    for _ in range(1500):
        op = rnd.random()
        try:
            if op < 0.25:
                s = book.acquire()
                assert s not in length and book.length(s) == 0
                length[s] = 0
            elif op < 0.85 and length:
                some = rnd.sample(sorted(length), rnd.randint(1, len(length)))
                n = rnd.choice([1, 1, 1, 9, 64, 130])
                if n == 1:
                    book.reserve_each(some, 1)
                    book.advance_each(some, 1)
                    for s in some:
                        length[s] += 1
                else:
                    book.reserve(some[0], n)
                    book.advance(some[0], n)
                    length[some[0]] += n
            elif length:
                s = rnd.choice(sorted(length))
                book.release(s)
                del length[s]
        except host.CacheFull:
            pass                                # refused; slots that reserve_each served before it failed keep their page
        book.check()
        assert book.lengths(sorted(length)) == [length[s] for s in sorted(length)]
        for s in length:
            n = book.length(s)
            full, win = book.pages_of(0, s), book.pages_of(1, s)
            need = -(-n // 64)
            assert sorted(full)[:need] == list(range(need)) and len(full) <= need + 1
            first = max(0, n - 100 + 1) // 64
            assert all(p >= first for p in win) and (n == 0 or (n - 1) // 64 in win)
            assert all(tables[0][s, p] == pid for p, pid in full.items())
            assert all(tables[1][s, p] == pid for p, pid in win.items())
    with pytest.raises(host.CacheError, match="not held"):
        book.release(next(s for s in range(slots) if s not in length))
    for s in list(length):
        book.release(s)
    book.check()
    assert book.free_slots == slots and book.free_pages(0) == n_pages and book.free_pages(1) == n_pages
