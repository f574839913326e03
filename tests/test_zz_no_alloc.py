"""The attention entry point that allocates nothing, called through its exported C symbol.

Some callers cannot allocate device memory when they need attention (a serving loop in
which cudaMalloc is forbidden or would stall the device, a plug-in running inside another
framework's stream, a process whose pool is already handed out) and have no scratch
buffer to pass.  ``ssb_attention_decode_static`` keeps the scratch of the split-key
kernel inside the library image instead.  This test binds the symbol with ctypes, as such
a caller would, and checks its output against the ordinary entry point on two calls in a
row: the arrays keep the first call's contents, and the second call must not be disturbed
by them.  It also checks that a request beyond the built-in scratch is refused.

Collected last on purpose (the file name sorts after every other test file), so that a
run that stops at the first failure has already run everything else.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bind():
    from supersonic_b200.csrc import build
    lib = ctypes.CDLL(build.build_library("attention_decode_static"))
    fn = lib.ssb_attention_decode_static
    fn.restype = c_int
    lib.ssb_attention_decode_static_limits.restype = None
    return lib, fn


def call(fn, q, k, v, pos, slot, table, out, n_q, n_kv, hd, window, scale, n_splits):
    p = lambda t: c_void_p(t.data_ptr())
    return fn(p(q), c_int(q.stride(0)), p(k), p(v), p(pos), p(slot), p(table), c_int(table.shape[1]), p(out),
              c_int(out.stride(0)), c_int(q.shape[0]), c_int(n_q), c_int(n_kv), c_int(hd), c_int(6),
              c_int(window or 0), c_float(scale), c_int(n_splits),
              c_void_p(torch.cuda.current_stream().cuda_stream))


def make_case(seed, n_q, n_kv, hd, n_seqs):
    g = torch.Generator(device=DEV).manual_seed(seed)
    n_pages = 6 * n_seqs
    k = torch.randn(n_pages, n_kv, 64, hd, device=DEV, generator=g).bfloat16()
    v = torch.randn(n_pages, n_kv, 64, hd, device=DEV, generator=g).bfloat16()
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32).view(n_seqs, 6).to(DEV)
    pos = torch.randint(0, 6 * 64, (n_seqs,), generator=torch.Generator().manual_seed(seed + 1)).to(torch.int32).to(DEV)
    slot = torch.arange(n_seqs, dtype=torch.int32, device=DEV)
    q = torch.randn(n_seqs, (n_q + 2 * n_kv) * hd, device=DEV, generator=g).bfloat16()
    return q, k, v, pos, slot, table


def test_static_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from supersonic_b200.csrc import ops
    lib, fn = bind()
    torch.cuda.set_device(0)
    # two different problems back to back: the second runs over what the first left behind
    for seed, (n_q, n_kv, hd, n_seqs, n_splits, window) in enumerate([(8, 2, 128, 5, 4, None),
                                                                       (6, 2, 48, 7, 6, 150)]):
        q, k, v, pos, slot, table = make_case(40 + seed, n_q, n_kv, hd, n_seqs)
        scale = 1 / math.sqrt(hd)
        nf, nc = ops.attention_decode_scratch(n_seqs, n_q, n_kv, hd, n_splits)
        want = torch.empty(n_seqs, n_q * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(q, k, v, pos, slot, table, want, n_q, n_kv, hd, 6, window, scale, n_splits,
                             torch.empty(nf, device=DEV), torch.zeros(nc, dtype=torch.int32, device=DEV))
        for _ in range(2):
            got = torch.full_like(want, 3.0)
            rc = call(fn, q, k, v, pos, slot, table, got, n_q, n_kv, hd, window, scale, n_splits)
            assert rc == 0
            torch.cuda.synchronize()
            torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_static_entry_point_refuses_what_its_scratch_cannot_hold():
    lib, fn = bind()
    floats, counters = c_longlong(0), c_int(0)
    lib.ssb_attention_decode_static_limits(ctypes.byref(floats), ctypes.byref(counters))
    assert floats.value == 2 * 1024 * 1024 and counters.value == 16 * 1024
    n_q, n_kv, hd, n_seqs, n_splits = 32, 8, 128, 64, 16          # 64*32*16*130 floats > 2 Mi
    assert n_seqs * n_q * n_splits * (hd + 2) > floats.value
    q, k, v, pos, slot, table = make_case(50, n_q, n_kv, hd, n_seqs)
    out = torch.full((n_seqs, n_q * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = call(fn, q, k, v, pos, slot, table, out, n_q, n_kv, hd, None, 0.1, n_splits)
    torch.cuda.synchronize()
    assert rc == 2005 and torch.all(out == 7.0)                   # refused, nothing launched
    assert call(fn, q, k, v, pos, slot, table, out, n_q, n_kv, hd, None, 0.1, 4) == 0   # 4 splits fit
    torch.cuda.synchronize()
    assert not torch.any(out == 7.0)


def test_static_entry_point_checks_sizes_before_it_enqueues_anything():
    """Sizes the kernel refuses (more than 64 splits, a head size above 256) are refused by the entry
    point itself with the size error, not after its counters were cleared on the stream."""
    lib, fn = bind()
    n_q, n_kv, hd, n_seqs = 4, 2, 64, 2
    q, k, v, pos, slot, table = make_case(60, n_q, n_kv, hd, n_seqs)
    out = torch.full((n_seqs, n_q * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    assert call(fn, q, k, v, pos, slot, table, out, n_q, n_kv, hd, None, 0.1, 65) == 2002
    assert call(fn, q, k, v, pos, slot, table, out, n_q, n_kv, 272, None, 0.1, 2) == 2002
    assert call(fn, q, k, v, pos, slot, table, out, 5, 2, hd, None, 0.1, 2) == 2002
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)
