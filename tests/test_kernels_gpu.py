"""Each plain kernel alone against a PyTorch float32 statement of the same operation, at
sizes other than the tiny models' (odd widths, several pages, windows)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from supersonic_b200.csrc import ops as o
    return o


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(301, 72, device=DEV, generator=g).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.full((5, 72), 7.0, device=DEV)
    ops().embed(ids, table, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype,wdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                          (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("hidden", [72, 1000, 4096])
def test_rmsnorm(dtype, wdtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(9, hidden, device=DEV, generator=g) * 3
    w = (1 + 0.1 * torch.randn(hidden, device=DEV, generator=g)).to(wdtype)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    for r in (None, rows):
        src = x if r is None else x[r.long()]
        out = torch.empty(src.shape, dtype=dtype, device=DEV)
        ops().rmsnorm(x, w, 1e-5, out, r)
        ref = src * torch.rsqrt((src * src).mean(-1, keepdim=True) + 1e-5) * w.float()
        torch.testing.assert_close(out.float(), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 301, 72), (7, 64, 200), (70, 130, 33), (129, 65, 257)])
def test_gemm_plain(dtype, M, N, K):
    g = torch.Generator(device=DEV).manual_seed(2)
    a = torch.randn(M, K, device=DEV, generator=g).to(dtype)
    w = torch.randn(N, K, device=DEV, generator=g).to(dtype)
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    ops().gemm_nt_plain(a, w, out)
    torch.testing.assert_close(out.double(), ref, atol=1e-4 if dtype == torch.float32 else 0.15, rtol=1e-2)
    acc = torch.ones(M, N, device=DEV)
    ops().gemm_nt_plain(a, w, acc, accumulate=True)
    torch.testing.assert_close(acc.double(), ref + 1, atol=1e-4, rtol=1e-5)
    out32 = torch.empty(M, N, device=DEV)
    ops().gemm_nt_plain(a, w, out32)
    torch.testing.assert_close(out32.double(), ref, atol=1e-4, rtol=1e-5)
    # a row-strided input (a slice of a wider buffer) gives the same result
    wide = torch.zeros(M, K + 5, dtype=dtype, device=DEV)
    wide[:, :K] = a
    out2 = torch.empty(M, N, device=DEV)
    ops().gemm_nt_plain(wide[:, :K], w, out2)
    assert torch.equal(out2, out32)


def _paged(n_pages, n_kv, hd, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    k = torch.randn(n_pages, n_kv, 64, hd, device=DEV, generator=g).to(dtype)
    v = torch.randn(n_pages, n_kv, 64, hd, device=DEV, generator=g).to(dtype)
    return k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,hd,rot", [(4, 2, 16, 16), (3, 1, 48, 48), (5, 5, 32, 16), (2, 1, 32, 0)])
def test_rope_append(dtype, n_q, n_kv, hd, rot):
    g = torch.Generator(device=DEV).manual_seed(3)
    T = 6
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV, generator=g).to(dtype)
    before = qkv.clone()
    pos = torch.tensor([0, 63, 64, 130, 5, 1], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 0, 0, 1, -1, 1], dtype=torch.int32, device=DEV)   # one padding row
    table = torch.tensor([[3, 1, 9], [4, 0, 2]], dtype=torch.int32, device=DEV)
    k, v = _paged(10, n_kv, hd, dtype, 4)
    k0, v0 = k.clone(), v.clone()
    half = rot // 2
    ang = torch.arange(200, device=DEV, dtype=torch.float64)[:, None] * \
        (1.0 / 10000 ** (torch.arange(max(half, 1), device=DEV, dtype=torch.float64) / max(half, 1)))[None, :half]
    cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    ops().rope_append(qkv, cos if rot else None, sin if rot else None, pos, slot, table, k, v,
                      n_q, n_kv, hd, rot, 6, True)
    for t in range(T):
        s, p = int(slot[t]), int(pos[t])
        x = before[t].float().view(n_q + 2 * n_kv, hd)
        if s < 0:
            assert torch.equal(qkv[t], before[t])
            continue
        want = x.clone()
        if rot:
            c, sn = cos[p], sin[p]
            r = x[: n_q + n_kv]
            want[: n_q + n_kv, :half] = r[:, :half] * c - r[:, half:rot] * sn
            want[: n_q + n_kv, half:rot] = r[:, :half] * sn + r[:, half:rot] * c
        torch.testing.assert_close(qkv[t].float().view(-1, hd), want.to(dtype).float(), **tol(dtype))
        page = int(table[s, p // 64])
        assert torch.equal(k[page, :, p % 64], qkv[t].view(-1, hd)[n_q:n_q + n_kv])
        assert torch.equal(v[page, :, p % 64], before[t].view(-1, hd)[n_q + n_kv:])
    touched = torch.zeros(10, 64, dtype=torch.bool, device=DEV)
    for t in range(T):
        if int(slot[t]) >= 0:
            touched[int(table[int(slot[t]), int(pos[t]) // 64]), int(pos[t]) % 64] = True
    kt, k0t, vt, v0t = (x.transpose(1, 2) for x in (k, k0, v, v0))         # [page, token, head, dim]
    assert torch.equal(kt[~touched], k0t[~touched]) and torch.equal(vt[~touched], v0t[~touched])


def _attention_reference(q, k, v, pos, slot, table, n_q, n_kv, hd, window, scale):
    out = torch.zeros(q.shape[0], n_q * hd, dtype=torch.float64, device=q.device)
    for t in range(q.shape[0]):
        s, p = int(slot[t]), int(pos[t])
        if s < 0:
            continue
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1, device=q.device)
        pages = table[s, js // 64].long()
        kk, vv = k[pages, :, js % 64].double(), v[pages, :, js % 64].double()      # [n, n_kv, hd]
        qq = q[t, : n_q * hd].double().view(n_q, hd)
        for h in range(n_q):
            sc = (kk[:, h // (n_q // n_kv)] @ qq[h]) * scale
            out[t, h * hd:(h + 1) * hd] = torch.softmax(sc, 0) @ vv[:, h // (n_q // n_kv)]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,hd,window", [(4, 2, 16, None), (3, 1, 48, None), (6, 2, 128, 100),
                                                (2, 2, 256, None), (8, 2, 64, 64)])
def test_attention_plain(dtype, n_q, n_kv, hd, window):
    g = torch.Generator(device=DEV).manual_seed(5)
    pos = torch.tensor([0, 1, 63, 64, 127, 128, 300, 299, 17], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 0, 0, 0, 1, 1, 1, 2, -1], dtype=torch.int32, device=DEV)
    perm = torch.randperm(15, generator=torch.Generator().manual_seed(6)).to(torch.int32)
    table = perm.view(3, 5).to(DEV)
    k, v = _paged(15, n_kv, hd, dtype, 7)
    ld = (n_q + 2 * n_kv) * hd
    q = torch.randn(len(pos), ld, device=DEV, generator=g).to(dtype)
    out = torch.full((len(pos), n_q * hd), 5.0, dtype=dtype, device=DEV)
    scale = 1 / math.sqrt(hd)
    ops().attention_plain(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, window, scale)
    ref = _attention_reference(q, k, v, pos, slot, table, n_q, n_kv, hd, window, scale)
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    assert torch.all(out[-1] == 0)                                      # padding row


def test_attention_finds_a_far_key_and_the_windows_edge():
    """One key among hundreds carries nearly all the weight: reading a neighbouring row, a
    wrong page or a key just outside the window changes the output completely."""
    n_q = n_kv = 1
    hd = 32
    k = torch.zeros(8, 1, 64, hd, device=DEV)
    v = torch.zeros(8, 1, 64, hd, device=DEV)
    table = torch.tensor([[5, 2, 7, 0, 3, 1]], dtype=torch.int32, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(8)
    for p in range(330):
        page = int(table[0, p // 64])
        k[page, 0, p % 64] = 0.01 * torch.randn(hd, device=DEV, generator=g)
        v[page, 0, p % 64, 0] = float(p)                                # value = its own position
    needle = 131
    k[int(table[0, needle // 64]), 0, needle % 64] = 4.0
    q = torch.full((1, hd), 4.0, device=DEV)
    pos = torch.tensor([329], dtype=torch.int32, device=DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(1, hd, device=DEV)
    for window, sees in ((None, True), (329 - needle + 1, True), (329 - needle, False)):
        ops().attention_plain(q, k, v, pos, slot, table, out, 1, 1, hd, 6, window, 1.0)
        if sees:
            assert abs(out[0, 0].item() - needle) < 1e-3
        else:
            lo = 329 - window + 1
            assert abs(out[0, 0].item() - (lo + 329) / 2) < 2.0          # near-uniform over the window


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_and_add(dtype):
    g = torch.Generator(device=DEV).manual_seed(9)
    gu = (3 * torch.randn(5, 2 * 200, device=DEV, generator=g)).to(dtype)
    z = torch.empty(5, 200, dtype=dtype, device=DEV)
    ops().swiglu(gu, z)
    gg, uu = gu[:, :200].float(), gu[:, 200:].float()
    torch.testing.assert_close(z.float(), (gg / (1 + torch.exp(-gg)) * uu).to(dtype).float(), **tol(dtype))
    acc = torch.ones(5, 200, device=DEV)
    ops().add_into(acc, z)
    torch.testing.assert_close(acc, 1 + z.float())


def test_argmax_lowest_index_wins():
    lg = torch.randn(6, 128256, device=DEV, generator=torch.Generator(device=DEV).manual_seed(10))
    lg[0, 77] = lg[0, 99000] = 50.0
    lg[1, 128255] = 60.0
    lg[2, :] = -float("inf")
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops().argmax(lg, out)
    assert out[0] == 77 and out[1] == 128255 and out[2] == 0
    assert torch.equal(out[3:].long(), lg[3:].argmax(-1))
    view = torch.randn(4, 700, device=DEV)[:, :301]                     # a row stride that is not the width
    o4 = torch.empty(4, dtype=torch.int32, device=DEV)
    ops().argmax(view, o4)
    assert torch.equal(o4.long(), view.argmax(-1))


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 0, 1.0), (0.7, 40, 1.0),
                                                     (1.0, 0, 0.9), (1.3, 25, 0.6)])
def test_sample_follows_the_reference_rule(temperature, top_k, top_p):
    """The drawn token is the one whose interval of the running sum (index order, over the
    kept tokens) holds u * kept mass; u comes from each row's own xorshift64 state."""
    import numpy as np
    import plain_llama as pl
    n, vocab = 12, 3001
    lg = 3 * torch.randn(n, vocab, device=DEV, generator=torch.Generator(device=DEV).manual_seed(11))
    seeds = [0x9E3779B97F4A7C15 * (i + 1) % (1 << 63) for i in range(n)]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    u = torch.empty(n, device=DEV)
    ops().sample(lg, temperature, top_k, top_p, None, state, out, u)
    for i in range(n):
        x = seeds[i]
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF; x ^= x >> 7; x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        assert int(state[i]) & 0xFFFFFFFFFFFFFFFF == x                  # the state moved one step
        assert abs(u[i].item() - (x >> 40) / 2 ** 24) < 1e-7
        p = pl.sampling_distribution(lg[i].double().cpu().numpy(), temperature, top_k, top_p)
        cdf = np.cumsum(p)
        t = int(out[i])
        assert p[t] > 0, "a token outside the kept set was drawn"
        lo, hi = cdf[t] - p[t], cdf[t]
        assert lo - 1e-4 <= u[i].item() <= hi + 1e-4
    # the same states draw the same tokens whatever rows they share a launch with
    state2 = torch.tensor(seeds[:3], dtype=torch.int64, device=DEV)
    out2 = torch.empty(3, dtype=torch.int32, device=DEV)
    ops().sample(lg[:3].contiguous(), temperature, top_k, top_p, None, state2, out2)
    assert torch.equal(out2, out[:3])


@pytest.mark.parametrize("vocab,temperature", [(128256, 1.0), (50021, 0.3), (2049, 1.7)])
def test_sample_by_temperature_alone_reads_the_row_in_stretches(vocab, temperature):
    """Without a cut the row is not held but read twice, in stretches of 2,048 logits per block of the
    cluster; rows here have their weight in a few far-apart places, whole stretches without any
    (minus infinity), or none at all."""
    import numpy as np
    import plain_llama as pl
    n = 40
    g = torch.Generator(device=DEV).manual_seed(vocab)
    lg = 2 * torch.randn(n, vocab, device=DEV, generator=g)
    lg[0, :] = -float("inf")                                            # nothing to draw from: token 0
    lg[1, : vocab // 2] = -float("inf")                                 # the first blocks of the cluster hold nothing
    lg[2, vocab // 3:] = -float("inf")
    lg[3, 5] = lg[3, vocab - 1] = 40.0                                  # two tokens share all the weight, at both ends
    lg[4, vocab // 2 + 1] = 60.0
    lg[5, :] = -float("inf"); lg[5, vocab - 3] = 1.0
    lg[6, 2048:] = -float("inf"); lg[6, :2040] = -float("inf")          # eight tokens at the end of the first stretch
    seeds = [0x9E3779B97F4A7C15 * (i + 3) % (1 << 63) for i in range(n)]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    u = torch.empty(n, device=DEV)
    ops().sample(lg, temperature, 0, 1.0, None, state, out, u)
    assert int(out[0]) == 0
    for i in range(1, n):
        p = pl.sampling_distribution(lg[i].double().cpu().numpy(), temperature, 0, 1.0)
        cdf = np.cumsum(p)
        t = int(out[i])
        assert p[t] > 0, f"row {i}: token {t} has no weight"
        assert cdf[t] - p[t] - 1e-4 <= u[i].item() <= cdf[t] + 1e-4, f"row {i}"
    # one row alone draws what it drew among the others
    state2 = torch.tensor(seeds[7:8], dtype=torch.int64, device=DEV)
    out2 = torch.empty(1, dtype=torch.int32, device=DEV)
    ops().sample(lg[7:8].contiguous(), temperature, 0, 1.0, None, state2, out2)
    assert int(out2[0]) == int(out[7])


@pytest.mark.parametrize("vocab", [128256, 40003])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.7, 40, 1.0), (1.0, 0, 0.9), (1.3, 25, 0.6), (1.0, 1, 1.0),
                                                     (0.5, 0, 0.01), (1.0, 3000, 0.999)])
def test_sample_with_cuts_at_a_large_vocabulary(vocab, temperature, top_k, top_p):
    """The cuts are found a byte of the key at a time over a cluster that holds the row: rows here have
    many tokens tied at a cut (logits on a grid of halves: all of them are kept), all their weight on one
    token, weight only far from the row's start, and ordinary random logits."""
    import numpy as np
    import plain_llama as pl
    n = 24
    g = torch.Generator(device=DEV).manual_seed(vocab + top_k)
    lg = 2 * torch.randn(n, vocab, device=DEV, generator=g)
    lg[0] = (lg[0] * 2).round() / 2                                     # ties everywhere
    lg[1] = (lg[1] * 2).round() / 2; lg[1, 7] = lg[1, vocab - 9] = 9.0  # two tied at the top
    lg[2, vocab // 2] = 80.0                                            # one token holds everything
    lg[3, : vocab - 100] = -float("inf")                                # only the last block of the cluster has weight
    lg[4, :] = 1.25                                                     # every token tied with every other
    lg[6, :] = -float("inf")                                            # nothing to draw from: token 0
    seeds = [0x9E3779B97F4A7C15 * (i + 5) % (1 << 63) for i in range(n)]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    u = torch.empty(n, device=DEV)
    ops().sample(lg, temperature, top_k, top_p, None, state, out, u)
    assert int(out[6]) == 0
    for i in range(n):
        if i == 6:
            continue
        p = pl.sampling_distribution(lg[i].double().cpu().numpy(), temperature, top_k, top_p)
        cdf = np.cumsum(p)
        t = int(out[i])
        assert p[t] > 0, f"row {i}: token {t} lies outside the kept set"
        assert cdf[t] - p[t] - 1e-4 <= u[i].item() <= cdf[t] + 1e-4, f"row {i}"
    # the same draw again, and one row alone
    state2 = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    out2 = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(lg, temperature, top_k, top_p, None, state2, out2)
    assert torch.equal(out, out2)
    state3 = torch.tensor(seeds[5:6], dtype=torch.int64, device=DEV)
    out3 = torch.empty(1, dtype=torch.int32, device=DEV)
    ops().sample(lg[5:6].contiguous(), temperature, top_k, top_p, None, state3, out3)
    assert int(out3[0]) == int(out[5])


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.8, 20, 0.9)])
def test_sample_at_a_vocabulary_beyond_the_cluster_kernels(temperature, top_k, top_p):
    """More than 524,288 logits a row: one block per row walks the row itself."""
    import numpy as np
    import plain_llama as pl
    n, vocab = 3, 530001
    lg = 2 * torch.randn(n, vocab, device=DEV, generator=torch.Generator(device=DEV).manual_seed(4))
    seeds = [0x9E3779B97F4A7C15 * (i + 9) % (1 << 63) for i in range(n)]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    u = torch.empty(n, device=DEV)
    ops().sample(lg, temperature, top_k, top_p, None, state, out, u)
    for i in range(n):
        p = pl.sampling_distribution(lg[i].double().cpu().numpy(), temperature, top_k, top_p)
        cdf = np.cumsum(p)
        t = int(out[i])
        assert p[t] > 0
        assert cdf[t] - p[t] - 1e-4 <= u[i].item() <= cdf[t] + 1e-4


def test_sample_uses_slots_for_its_generator():
    lg = torch.randn(2, 500, device=DEV)
    state = torch.tensor([11, 22, 33, 44], dtype=torch.int64, device=DEV) * 0x2545F4914F6CDD1D % (1 << 62)
    before = state.clone()
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    ops().sample(lg, 1.0, 0, 1.0, slots, state, out)
    assert state[0] == before[0] and state[2] == before[2]
    assert state[1] != before[1] and state[3] != before[3]


def test_kernels_refuse_what_they_cannot_do():
    from supersonic_b200.csrc.ops import KernelError
    with pytest.raises(KernelError, match="CUDA"):
        ops().swiglu(torch.zeros(2, 4), torch.zeros(2, 2))
    with pytest.raises(KernelError, match="float32 or bfloat16"):
        ops().gemm_nt_plain(torch.zeros(2, 4, device=DEV, dtype=torch.float16),
                            torch.zeros(3, 4, device=DEV, dtype=torch.float16), torch.zeros(2, 3, device=DEV))
    with pytest.raises(KernelError, match="head_dim"):
        ops().attention_plain(torch.zeros(1, 1024, device=DEV), torch.zeros(1, 1, 64, 1024, device=DEV),
                              torch.zeros(1, 1, 64, 1024, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                              torch.zeros(1, dtype=torch.int32, device=DEV),
                              torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, 1024, device=DEV),
                              1, 1, 1024, 6, None, 1.0)


# ---- decode kernels -----------------------------------------------------------------------
@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("N,K", [(301, 72), (48, 200), (1000, 4096), (272, 1440)])
def test_skinny_gemm_store_and_accumulate(rows, N, K):
    g = torch.Generator(device=DEV).manual_seed(20)
    x = torch.randn(rows, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    ref = x.double() @ w.double().T
    out = torch.empty(rows, N, device=DEV)
    ops().skinny_gemm(x, w, out)
    torch.testing.assert_close(out.double(), ref, atol=2e-5 * math.sqrt(K), rtol=1e-4)
    ob = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
    ops().skinny_gemm(x, w, ob)
    torch.testing.assert_close(ob.double(), ref, atol=2e-2, rtol=2e-2)
    acc = torch.full((rows, N), 2.0, device=DEV)
    ops().skinny_gemm(x, w, acc, mode=1)
    torch.testing.assert_close(acc.double(), ref + 2, atol=2e-5 * math.sqrt(K), rtol=1e-4)
    plain = torch.empty(rows, N, device=DEV)
    ops().gemm_nt_plain(x, w, plain)
    torch.testing.assert_close(out, plain, atol=2e-5 * math.sqrt(K), rtol=1e-4)


@pytest.mark.parametrize("rows", [1, 5, 40])
def test_skinny_gemm_swiglu(rows):
    g = torch.Generator(device=DEV).manual_seed(22)
    K, inter = 72, 200
    x = torch.randn(rows, K, device=DEV, generator=g).bfloat16()
    gate = (torch.randn(inter, K, device=DEV, generator=g) / 4).bfloat16()
    up = (torch.randn(inter, K, device=DEV, generator=g) / 4).bfloat16()
    from supersonic_b200.csrc.fast_sets import FastKernels
    packed, layout = FastKernels().pack_gate_up(gate, up)
    assert layout == "interleaved" and torch.equal(packed[:8], gate[:8]) and torch.equal(packed[8:16], up[:8])
    out = torch.empty(rows, inter, dtype=torch.bfloat16, device=DEV)
    ops().skinny_gemm(x, packed, out, mode=2)
    gg, uu = x.double() @ gate.double().T, x.double() @ up.double().T
    torch.testing.assert_close(out.double(), gg / (1 + torch.exp(-gg)) * uu, atol=2e-2, rtol=2e-2)
    # the unfused way over the same packed weights agrees
    gu = torch.empty(rows, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops().gemm_nt_plain(x, packed, gu)
    z = torch.empty(rows, inter, dtype=torch.bfloat16, device=DEV)
    ops().swiglu(gu, z, interleaved=True)
    torch.testing.assert_close(out.float(), z.float(), atol=2e-2, rtol=2e-2)


def _decode_attention(kind, q, k, v, pos, slot, table, out, n_q, n_kv, hd, window, scale, n_splits, max_pages,
                      cos=None, sin=None, poison=True):
    """kind 1: the CUDA-core kernel with ``n_splits`` splits; kind 2: the tensor-core kernel on its
    persistent grid with chunks of ceil(max_pages / n_splits) pages (so that the longest sequence is cut
    into about ``n_splits`` chunks); kind 3: the tensor-core kernel with a sequence's chunks as a
    thread-block cluster of 2, 4 or 8 blocks (the power of two from ``n_splits`` up) that merges through
    its shared memory.  Returns the counters, which every launch must leave zero."""
    B = q.shape[0]
    cluster = 0
    if kind == 3:
        cluster = 2 if n_splits <= 2 else (4 if n_splits <= 4 else 8)
        while cluster >= 2 and (B * n_kv * cluster > ops().attention_decode_chunked_blocks(B, n_q, n_kv, hd, cos is not None)
                                or B * n_kv > ops().attention_decode_chunked_clusters(n_q, n_kv, hd, cos is not None, cluster)):
            cluster //= 2                                                # the clusters' blocks must all fit the device at once
        if cluster < 2:
            pytest.skip("too many (sequence, kv head) pairs for clusters")
    if kind == 1:
        nf, nc = ops().attention_decode_scratch(B, n_q, n_kv, hd, n_splits)
    else:
        chunk = -(-max_pages // n_splits)
        max_chunks = -(-max_pages // chunk)
        nf, nc = ops().attention_decode_chunked_scratch(B, n_q, n_kv, hd, max_chunks)
    scratch = torch.full((max(nf, 1),), float("nan") if poison else 0.0, device=DEV)
    counters = torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV)
    for _ in range(2):                                                   # counters are left ready for reuse
        out.fill_(5.0)
        if kind == 1:
            ops().attention_decode(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, window, scale, n_splits,
                                   scratch, counters, cos=cos, sin=sin)
        else:
            ops().attention_decode_chunked(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, window, scale, chunk,
                                           max_chunks, scratch, counters, cos=cos, sin=sin, cluster=cluster)
        if cos is not None:
            break                                                        # a fused launch appends: once only
    return counters


@pytest.mark.parametrize("n_q,n_kv,hd,window", [(4, 2, 16, None), (3, 1, 48, None), (32, 8, 128, None),
                                                (6, 2, 128, 100), (2, 2, 256, None), (8, 1, 64, 64),
                                                (5, 5, 80, None), (12, 1, 128, None), (32, 2, 64, 150)])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
@pytest.mark.parametrize("kind", [1, 2, 3])
def test_attention_decode(n_q, n_kv, hd, window, n_splits, kind):
    if kind >= 2 and (hd not in (64, 128) or n_q // n_kv > 16):
        pytest.skip("the tensor-core kernel takes head_dim 64/128 and at most 16 query heads per kv head")
    g = torch.Generator(device=DEV).manual_seed(23)
    pos = torch.tensor([0, 63, 64, 300, 299, 17, 128], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 1, 2, 3, 4, -1, 5], dtype=torch.int32, device=DEV)
    table = torch.randperm(30, generator=torch.Generator().manual_seed(24)).to(torch.int32).view(6, 5).to(DEV)
    k, v = _paged(30, n_kv, hd, torch.bfloat16, 25)
    q = torch.randn(len(pos), (n_q + 2 * n_kv) * hd, device=DEV, generator=g).bfloat16()
    scale = 1 / math.sqrt(hd)
    ref = _attention_reference(q, k, v, pos, slot, table, n_q, n_kv, hd, window, scale)
    out = torch.empty((len(pos), n_q * hd), dtype=torch.bfloat16, device=DEV)
    counters = _decode_attention(kind, q, k, v, pos, slot, table, out, n_q, n_kv, hd, window, scale, n_splits, 5)
    torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)
    assert torch.all(out[5] == 0) and torch.all(counters == 0)
    plain = torch.empty_like(out)
    ops().attention_plain(q, k, v, pos, slot, table, plain, n_q, n_kv, hd, 6, window, scale)
    torch.testing.assert_close(out.float(), plain.float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("kind", [1, 2])
@pytest.mark.parametrize("n_splits,slope", [(13, 0.02), (21, -0.02), (16, 0.0)])
def test_attention_decode_merges_many_splits(kind, n_splits, slope):
    """More splits than the merge takes in one go (eight), over 21 pages, with scores that climb
    or fall along the keys so that the maximum moves from one group of splits to the next."""
    n_q, n_kv, hd, n = 8, 2, 128, 1300
    g = torch.Generator(device=DEV).manual_seed(26)
    n_pages = (n + 63) // 64
    table = torch.randperm(2 * n_pages, generator=torch.Generator().manual_seed(27)).to(torch.int32).view(2, n_pages).to(DEV)
    k, v = _paged(2 * n_pages, n_kv, hd, torch.bfloat16, 28)
    ramp = (slope * torch.arange(n_pages * 64, device=DEV, dtype=torch.float32) * math.sqrt(hd)).bfloat16()
    for s in range(2):
        for pg in range(n_pages):
            k[int(table[s, pg]), :, :, 0] = ramp[pg * 64:(pg + 1) * 64][None, :]
    pos = torch.tensor([n - 1, 777], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    q = 0.3 * torch.randn(2, (n_q + 2 * n_kv) * hd, device=DEV, generator=g).bfloat16()
    q[:, 0:n_q * hd:hd] = 1.0                                          # every head looks along the ramp
    scale = 1 / math.sqrt(hd)
    out = torch.empty(2, n_q * hd, dtype=torch.bfloat16, device=DEV)
    counters = _decode_attention(kind, q, k, v, pos, slot, table, out, n_q, n_kv, hd, None, scale, n_splits, n_pages)
    ref = _attention_reference(q, k, v, pos, slot, table, n_q, n_kv, hd, None, scale)
    torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)
    assert torch.all(counters == 0)


def test_round_and_clear():
    g = torch.Generator(device=DEV).manual_seed(33)
    sums = torch.randn(37, 264, device=DEV, generator=g)
    want = sums.bfloat16()
    wide = torch.full((37, 272), 3.0, dtype=torch.bfloat16, device=DEV)
    ops().round_and_clear(sums, wide[:, :264])
    assert torch.equal(wide[:, :264], want) and torch.all(wide[:, 264:] == 3.0) and torch.all(sums == 0)


@pytest.mark.parametrize("rows", [8, 12, 16, 17, 40, 64, 65, 130, 300])
@pytest.mark.parametrize("N,K", [(6144, 4096), (1000, 1088)])
def test_fast_linear_picks_a_kernel_for_every_row_count(rows, N, K):
    """The bfloat16 kernel set's projection at row counts on both sides of every threshold: stored
    as bfloat16, and added into a float32 residual; twice in a row (scratch is left as it was found)."""
    from supersonic_b200.csrc.fast_sets import FastKernels
    ks = FastKernels()
    g = torch.Generator(device=DEV).manual_seed(34)
    x = torch.randn(rows, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    ref = x.double() @ w.double().T
    for _ in range(2):
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
        ks.linear(x, w, out)
        torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)
        res = torch.full((rows, N), 2.0, device=DEV)
        ks.linear(x, w, res, accumulate=True)
        torch.testing.assert_close(res.double(), ref + 2, atol=2e-3, rtol=1e-3)
    ops().check_device_errors()


# ---- prefill GEMM on tcgen05 ------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (65, 128, 200), (200, 304, 72), (300, 1000, 4096),
                                   (1024, 512, 1024), (129, 8, 64),
                                   (4400, 520, 128)])       # 18 row tiles of 256: a band of 16 and one of 2
@pytest.mark.parametrize("tile_n", [64, 128, 256, 512])         # 512: tiles of 256 x 256 on SM pairs
def test_gemm_tc(M, N, K, tile_n):
    g = torch.Generator(device=DEV).manual_seed(30)
    a = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    ref = a.double() @ w.double().T
    out = torch.full((M, N), 9.0, device=DEV)
    ops().gemm_tc(a, w, out, tile_n=tile_n)
    ops().check_device_errors()
    torch.testing.assert_close(out.double(), ref, atol=2e-5 * math.sqrt(K), rtol=1e-4)
    ob = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops().gemm_tc(a, w, ob, tile_n=tile_n)
    torch.testing.assert_close(ob.double(), ref, atol=2e-2, rtol=2e-2)
    acc = torch.full((M, N), 2.0, device=DEV)
    ops().gemm_tc(a, w, acc, mode=1, tile_n=tile_n)
    torch.testing.assert_close(acc.double(), ref + 2, atol=2e-5 * math.sqrt(K), rtol=1e-4)
    ops().check_device_errors()
    # a row-strided input (a slice of a wider buffer) gives the same result
    wide = torch.zeros(M, K + 8, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = a
    out2 = torch.empty(M, N, device=DEV)
    ops().gemm_tc(wide[:, :K], w, out2, tile_n=tile_n)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M,N,K,tile_n,splits", [(130, 512, 4096, 256, 8), (300, 1000, 1088, 128, 3),
                                                 (128, 4096, 14336, 256, 16), (65, 264, 640, 64, 7)])
def test_gemm_tc_with_k_cut_into_parts(M, N, K, tile_n, splits):
    """Few output tiles: every tile's K range is cut into parts that add with float atomics (also a
    number of parts that does not divide the k-blocks, and more parts than k-blocks allow)."""
    g = torch.Generator(device=DEV).manual_seed(32)
    a = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    ref = a.double() @ w.double().T
    base = torch.randn(M, N, device=DEV, generator=g)
    acc = base.clone()
    for _ in range(2):
        ops().gemm_tc(a, w, acc, mode=1, tile_n=tile_n, splits=splits)
    ops().check_device_errors()
    torch.testing.assert_close(acc.double(), base.double() + 2 * ref, atol=4e-5 * math.sqrt(K), rtol=1e-4)
    from supersonic_b200.csrc.ops import KernelError
    with pytest.raises(KernelError):
        ops().gemm_tc(a, w, torch.empty(M, N, dtype=torch.bfloat16, device=DEV), tile_n=tile_n, splits=splits)


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """A bounded mbarrier wait at which nothing arrives gives up after about a second; the error
    word carries the role, ``check_device_errors`` raises once and clears it, and the next GEMM is right."""
    import time
    from supersonic_b200.csrc.ops import KernelError
    ops().check_device_errors()
    t0 = time.perf_counter()
    ops().tc_wait_probe(DEV)
    with pytest.raises(KernelError, match="bounded wait ran out in the TMA producer"):
        ops().check_device_errors()
    assert 0.2 < time.perf_counter() - t0 < 10.0
    ops().check_device_errors()                                         # cleared: no second report
    a = torch.randn(128, 256, device=DEV).bfloat16()
    w = torch.randn(64, 256, device=DEV).bfloat16()
    out = torch.empty(128, 64, device=DEV)
    ops().gemm_tc(a, w, out)
    ops().check_device_errors()
    torch.testing.assert_close(out.double(), a.double() @ w.double().T, atol=1e-3, rtol=1e-4)


def test_scratch_that_must_be_zero_between_uses_is_zeroed_after_a_reported_error():
    """A launch that gave up may leave arrival counters and partial sums half-way: when the error is
    reported, every kernel set alive puts its zero-between-uses buffers back to zero (and sets that
    were dropped are no longer called)."""
    from supersonic_b200.csrc.fast_sets import FastKernels
    from supersonic_b200.csrc.ops import KernelError
    ops().check_device_errors()
    kept, dropped = FastKernels(), FastKernels()
    counters = kept._buffer("attn_counters", 64, torch.int32, torch.device(DEV), zero=True)
    sums = kept._buffer("split_sums", 256, torch.float32, torch.device(DEV), zero=True)
    plain = kept._buffer("attn_partials", 256, torch.float32, torch.device(DEV))
    counters.fill_(3); sums.fill_(1.5); plain.fill_(7.0)
    del dropped
    ops().tc_wait_probe(DEV)
    with pytest.raises(KernelError, match="bounded wait ran out"):
        ops().check_device_errors()
    assert int(counters.abs().sum()) == 0 and float(sums.abs().sum()) == 0.0
    assert float(plain[0]) == 7.0                                        # ordinary scratch is left alone
    ops().check_device_errors()


@pytest.mark.parametrize("tile_n", [256, 512])
@pytest.mark.parametrize("M,inter,K", [(130, 200, 72), (256, 1024, 512), (700, 1160, 320)])
def test_gemm_tc_swiglu(M, inter, K, tile_n):
    g = torch.Generator(device=DEV).manual_seed(31)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    gate = (torch.randn(inter, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    up = (torch.randn(inter, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    from supersonic_b200.csrc.fast_sets import FastKernels
    packed, layout = FastKernels().pack_gate_up(gate, up)
    out = torch.empty(M, inter, dtype=torch.bfloat16, device=DEV)
    ops().gemm_tc(x, packed, out, mode=2, tile_n=tile_n)
    ops().check_device_errors()
    gg, uu = x.double() @ gate.double().T, x.double() @ up.double().T
    torch.testing.assert_close(out.double(), gg / (1 + torch.exp(-gg)) * uu, atol=2e-2, rtol=2e-2)


# ---- prefill attention ---------------------------------------------------------------------------
def _prefill_kernel(impl):
    return ops().attention_prefill_tc if impl == "tcgen05" else ops().attention_prefill


@pytest.mark.parametrize("impl", ["mma", "tcgen05"])
@pytest.mark.parametrize("n_q,n_kv,hd,window", [(8, 2, 128, None), (4, 4, 64, None), (6, 2, 128, 100),
                                                (3, 1, 64, 64), (2, 1, 128, 1), (3, 1, 128, None),
                                                (5, 5, 128, 70)])
def test_attention_prefill(n_q, n_kv, hd, window, impl):
    """A ragged batch: sequences that start at 0 and sequences that continue a cached prefix,
    lengths that end inside a page, on page borders and inside a tile; groups of one, odd and even
    numbers of query heads (the tcgen05 kernel pairs tiles of a group)."""
    g = torch.Generator(device=DEV).manual_seed(40)
    starts = [0, 0, 64, 37, 0, 200]
    news = [1, 150, 64, 91, 64, 130]
    n_seqs = len(starts)
    pages_per = 6
    table = torch.randperm(n_seqs * pages_per, generator=torch.Generator().manual_seed(41)).to(torch.int32)
    table = table.view(n_seqs, pages_per).to(DEV)
    k, v = _paged(n_seqs * pages_per, n_kv, hd, torch.bfloat16, 42)
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    T = cu[-1]
    q = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV, generator=g).bfloat16()
    slot = torch.arange(n_seqs, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    out = torch.full((T, n_q * hd), 5.0, dtype=torch.bfloat16, device=DEV)
    _prefill_kernel(impl)(q, k, v, torch.tensor(cu, dtype=torch.int32, device=DEV),
                          torch.tensor(starts, dtype=torch.int32, device=DEV), slot, table, out, max(news),
                          n_q, n_kv, hd, 6, window, scale)
    ops().check_device_errors()
    pos = torch.tensor([s + i for s, n in zip(starts, news) for i in range(n)], dtype=torch.int32, device=DEV)
    slot_tok = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32, device=DEV)
    ref = _attention_reference(q, k, v, pos, slot_tok, table, n_q, n_kv, hd, window, scale)
    torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)
    plain = torch.empty_like(out)
    ops().attention_plain(q, k, v, pos, slot_tok, table, plain, n_q, n_kv, hd, 6, window, scale)
    torch.testing.assert_close(out.float(), plain.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("impl", ["mma", "tcgen05"])
@pytest.mark.parametrize("slope", [0.05, 0.2, -0.05])
def test_attention_prefill_with_scores_that_drift(impl, slope):
    """Scores that climb (or fall) steadily along the keys: the running maximum moves a little in
    every block of keys, by less or by more than the step at which the tcgen05 kernel rescales."""
    hd, n = 128, 700
    g = torch.Generator(device=DEV).manual_seed(47)
    n_pages = (n + 63) // 64
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(48)).to(torch.int32).view(1, -1).to(DEV)
    k = torch.zeros(n_pages, 1, 64, hd, dtype=torch.bfloat16, device=DEV)
    v = torch.randn(n_pages, 1, 64, hd, device=DEV, generator=g).bfloat16()
    ramp = (slope * torch.arange(n, device=DEV, dtype=torch.float32)).bfloat16()
    for p0 in range(0, n, 64):
        m = min(64, n - p0)
        k[int(table[0, p0 // 64]), 0, :m, 0] = ramp[p0:p0 + m]
    q = 0.1 * torch.randn(n, 3 * hd, device=DEV, generator=g).bfloat16()
    q[:, 0] = 1.0
    out = torch.empty(n, hd, dtype=torch.bfloat16, device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    slot_tok = torch.zeros(n, dtype=torch.int32, device=DEV)
    _prefill_kernel(impl)(q, k, v, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                          torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                          table, out, n, 1, 1, hd, 6, None, 1.0)
    ops().check_device_errors()
    ref = _attention_reference(q, k, v, pos, slot_tok, table, 1, 1, hd, None, 1.0)
    torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("impl", ["mma", "tcgen05"])
def test_attention_prefill_finds_a_far_key(impl):
    """One key among hundreds carries the weight for the last query; its neighbours do not."""
    kernel = _prefill_kernel(impl)
    hd = 128
    k = torch.zeros(8, 1, 64, hd, dtype=torch.bfloat16, device=DEV)
    v = torch.zeros(8, 1, 64, hd, dtype=torch.bfloat16, device=DEV)
    table = torch.tensor([[5, 2, 7, 0, 3, 1]], dtype=torch.int32, device=DEV)
    for p in range(330):
        v[int(table[0, p // 64]), 0, p % 64, 0] = float(p % 128)          # exactly representable
    needle = 131
    k[int(table[0, needle // 64]), 0, needle % 64] = 2.0
    q = torch.zeros(330, 3 * hd, dtype=torch.bfloat16, device=DEV)
    q[329, :hd] = 2.0
    out = torch.empty(330, hd, dtype=torch.bfloat16, device=DEV)
    args = (torch.tensor([0, 330], dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
            torch.zeros(1, dtype=torch.int32, device=DEV), table, out, 330, 1, 1, hd, 6)
    kernel(q, k, v, *args, None, 1.0)
    assert abs(out[329, 0].item() - needle % 128) < 0.51
    kernel(q, k, v, *args, 329 - needle + 1, 1.0)       # the window's last key is the needle
    assert abs(out[329, 0].item() - needle % 128) < 0.51
    kernel(q, k, v, *args, 329 - needle, 1.0)           # one shorter: the needle is outside
    assert abs(out[329, 0].item() - needle % 128) > 10


@pytest.mark.parametrize("n_q,n_kv,hd,window", [(32, 8, 128, None), (4, 2, 64, None), (6, 2, 128, 100),
                                                (2, 1, 32, None), (8, 8, 256, None), (10, 1, 128, None),
                                                (32, 2, 64, 90)])
@pytest.mark.parametrize("n_splits", [1, 4, 8])
@pytest.mark.parametrize("kind", [1, 2, 3])
def test_attention_decode_with_rotation_and_append_inside(n_q, n_kv, hd, window, n_splits, kind):
    if kind >= 2 and (hd not in (64, 128) or n_q // n_kv > 16):
        pytest.skip("the tensor-core kernel takes head_dim 64/128 and at most 16 query heads per kv head")
    """The fused launch equals rope_append followed by attention_decode: output, and the key
    and value it leaves in the cache; positions include 0, page borders and a padding row."""
    g = torch.Generator(device=DEV).manual_seed(50)
    pos = torch.tensor([0, 63, 64, 300, 299, 17, 128], dtype=torch.int32, device=DEV)
    slot = torch.tensor([0, 1, 2, 3, 4, -1, 5], dtype=torch.int32, device=DEV)
    table = torch.randperm(30, generator=torch.Generator().manual_seed(51)).to(torch.int32).view(6, 5).to(DEV)
    k0, v0 = _paged(30, n_kv, hd, torch.bfloat16, 52)
    qkv0 = torch.randn(len(pos), (n_q + 2 * n_kv) * hd, device=DEV, generator=g).bfloat16()
    ang = torch.arange(400, device=DEV, dtype=torch.float64)[:, None] * \
        (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV, dtype=torch.float64) * 2 / hd))[None, :]
    cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    scale = 1 / math.sqrt(hd)
    # the two-step way
    qkv_a, ka, va = qkv0.clone(), k0.clone(), v0.clone()
    ops().rope_append(qkv_a, cos, sin, pos, slot, table, ka, va, n_q, n_kv, hd, hd, 6, True)
    want = torch.empty(len(pos), n_q * hd, dtype=torch.bfloat16, device=DEV)
    _decode_attention(1, qkv_a, ka, va, pos, slot, table, want, n_q, n_kv, hd, window, scale, n_splits, 5)
    # the fused way
    qkv_b, kb, vb = qkv0.clone(), k0.clone(), v0.clone()
    got = torch.full_like(want, 5.0)
    counters = _decode_attention(kind, qkv_b, kb, vb, pos, slot, table, got, n_q, n_kv, hd, window, scale, n_splits, 5,
                                 cos=cos, sin=sin)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(qkv_b, qkv0)                                       # the projection's output is not touched
    assert torch.equal(vb, va)                                            # values are copied as they are
    torch.testing.assert_close(kb.float(), ka.float(), atol=0, rtol=2 ** -7)   # keys: at most the last bit
    assert torch.all(got[5] == 0) and torch.all(counters == 0)


@pytest.mark.parametrize("rows", [1, 16, 17, 33, 64, 65, 100, 128])
@pytest.mark.parametrize("N,K,splits", [(304, 72, 1), (1000, 4096, 1), (1000, 4096, 5), (128, 640, 3), (272, 1440, 8)])
def test_gemv_tc(rows, N, K, splits):
    g = torch.Generator(device=DEV).manual_seed(70)
    x = torch.randn(rows, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    ref = x.double() @ w.double().T
    nf, nc = ops().gemv_tc_scratch(rows, N, splits)
    partials = torch.full((max(nf, 4),), float("nan"), device=DEV)
    counters = torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV)
    kw = dict(splits=splits, partials=partials, counters=counters)
    for _ in range(2):                                                   # the counters are left ready
        out = torch.full((rows, N), 9.0, device=DEV)
        ops().gemv_tc(x, w, out, **kw)
        ops().check_device_errors()
        torch.testing.assert_close(out.double(), ref, atol=2e-5 * math.sqrt(K), rtol=1e-4)
        assert torch.all(counters == 0)
    ob = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
    ops().gemv_tc(x, w, ob, **kw)
    torch.testing.assert_close(ob.double(), ref, atol=2e-2, rtol=2e-2)
    acc = torch.full((rows, N), 2.0, device=DEV)
    ops().gemv_tc(x, w, acc, mode=1, splits=splits)                      # float atomics when K is split
    torch.testing.assert_close(acc.double(), ref + 2, atol=2e-5 * math.sqrt(K), rtol=1e-4)
    again = torch.full((rows, N), 9.0, device=DEV)
    ops().gemv_tc(x, w, again, **kw)
    assert torch.equal(again, out)                                       # same sum order every time
    ops().check_device_errors()


@pytest.mark.parametrize("rows,splits", [(20, 1), (64, 3), (97, 1), (128, 2)])
def test_gemv_tc_swiglu(rows, splits):
    g = torch.Generator(device=DEV).manual_seed(71)
    K, inter = 576, 200
    x = torch.randn(rows, K, device=DEV, generator=g).bfloat16()
    gate = (torch.randn(inter, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    up = (torch.randn(inter, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    from supersonic_b200.csrc.fast_sets import FastKernels
    packed, layout = FastKernels().pack_gate_up(gate, up)
    nf, nc = ops().gemv_tc_scratch(rows, 2 * inter, splits)
    out = torch.empty(rows, inter, dtype=torch.bfloat16, device=DEV)
    ops().gemv_tc(x, packed, out, mode=2, splits=splits, partials=torch.empty(max(nf, 4), device=DEV),
                  counters=torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV))
    ops().check_device_errors()
    gg, uu = x.double() @ gate.double().T, x.double() @ up.double().T
    torch.testing.assert_close(out.double(), gg / (1 + torch.exp(-gg)) * uu, atol=2e-2, rtol=2e-2)


# ---- vector element-wise kernels ---------------------------------------------------------------------
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("hidden", [72, 1000, 4096, 8192])
def test_rmsnorm_vec_equals_plain(wdtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(80)
    x = torch.randn(70, hidden, device=DEV, generator=g) * 3
    w = (1 + 0.1 * torch.randn(hidden, device=DEV, generator=g)).to(wdtype)
    rows = torch.tensor([69, 0, 3, 3], dtype=torch.int32, device=DEV)
    for r in (None, rows):
        n = 70 if r is None else 4
        want = torch.empty(n, hidden, dtype=torch.bfloat16, device=DEV)
        got = torch.full((n, hidden), 9.0, dtype=torch.bfloat16, device=DEV)
        ops().rmsnorm(x, w, 1e-5, want, r)
        ops().rmsnorm_vec(x, w, 1e-5, got, r)
        # same formula; the sum of squares is added in another order
        torch.testing.assert_close(got.float(), want.float(), atol=0, rtol=2 ** -7)


@pytest.mark.parametrize("tile_n", [256, 512])
@pytest.mark.parametrize("n_q,n_kv,hd,K,T", [(3, 1, 128, 192, 300), (5, 2, 64, 264, 129), (9, 3, 64, 64, 513)])
def test_projection_with_rope_and_append_in_its_epilogue(n_q, n_kv, hd, K, T, tile_n):
    """gemm_tc_rope_append against float32: rotated queries in the output, rotated keys and plain
    values at each token's page and place; other cache rows, skipped rows' outputs and the output's
    spare columns untouched.  Widths end inside a tile of 256 columns and inside a tile of 128 rows."""
    g = torch.Generator(device=DEV).manual_seed(181)
    n_slots, max_pages = 3, (T + 63) // 64 + 1
    a = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn((n_q + 2 * n_kv) * hd, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    # three sequences that continue at different places; a cache row is written once
    slot = (torch.arange(T) % n_slots).to(torch.int32)
    pos = (torch.arange(T) // n_slots + torch.tensor([0, 37, 64])[slot.long()]).to(torch.int32)
    slot[5], slot[T - 1] = -1, -1
    slot, pos = slot.to(DEV), pos.to(DEV)
    n_pages = n_slots * max_pages
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(184)).to(torch.int32).view(n_slots, max_pages).to(DEV)
    n_pos = int(pos.max()) + 1
    ang = torch.arange(n_pos, device=DEV, dtype=torch.float64)[:, None] * \
        (1.0 / 500000 ** (torch.arange(hd // 2, device=DEV, dtype=torch.float64) * 2 / hd))[None, :]
    cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    k0, v0 = _paged(n_pages, n_kv, hd, torch.bfloat16, 185)
    kc, vc = k0.clone(), v0.clone()
    out = torch.full((T, n_q * hd + 8), 7.0, device=DEV, dtype=torch.bfloat16)
    ops().gemm_tc_rope_append(a, w, out, cos, sin, pos, slot, table, kc, vc, n_q, n_kv, hd, 6, tile_n=tile_n)
    ops().check_device_errors()
    sums = (a.double() @ w.double().T).view(T, n_q + 2 * n_kv, hd)
    lo, hi = sums[..., : hd // 2], sums[..., hd // 2:]
    c, sn = ang.cos()[pos.long()][:, None, :], ang.sin()[pos.long()][:, None, :]
    rot = torch.cat([lo * c - hi * sn, lo * sn + hi * c], dim=-1)
    live = slot >= 0
    tol = dict(atol=2e-2, rtol=2 ** -7)                      # one bfloat16 rounding of sums of size ~1
    torch.testing.assert_close(out[live, : n_q * hd].double(), rot[live, :n_q].reshape(-1, n_q * hd), **tol)
    assert (out[:, n_q * hd:] == 7.0).all() and (out[~live] == 7.0).all()
    want_k, want_v = k0.double(), v0.double()
    page = table[slot.clamp(min=0).long(), (pos >> 6).long()].long()
    for t in torch.nonzero(live).flatten().tolist():
        want_k[page[t], :, int(pos[t]) & 63] = rot[t, n_q: n_q + n_kv]
        want_v[page[t], :, int(pos[t]) & 63] = sums[t, n_q + n_kv:]
    torch.testing.assert_close(kc.double(), want_k, **tol)
    torch.testing.assert_close(vc.double(), want_v, **tol)
    untouched = torch.ones(n_pages, 64, dtype=torch.bool, device=DEV)
    untouched[page[live], (pos[live] & 63).long()] = False
    assert torch.equal(kc.transpose(1, 2)[untouched], k0.transpose(1, 2)[untouched])
    assert torch.equal(vc.transpose(1, 2)[untouched], v0.transpose(1, 2)[untouched])


@pytest.mark.parametrize("n_q,n_kv,hd", [(4, 2, 16), (3, 1, 48), (32, 8, 128), (5, 5, 64)])
def test_rope_append_vec_equals_plain(n_q, n_kv, hd):
    g = torch.Generator(device=DEV).manual_seed(81)
    T = 70
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd + 8, device=DEV, generator=g).bfloat16()     # a wider row stride
    pos = torch.randint(0, 5 * 64, (T,), generator=torch.Generator().manual_seed(82)).to(torch.int32).to(DEV)
    slot = torch.randint(-1, 3, (T,), generator=torch.Generator().manual_seed(83)).to(torch.int32).to(DEV)
    key = slot.long() * 1000 + pos.long()                                                    # a cache row is written once
    keep = torch.ones(T, dtype=torch.bool, device=DEV)
    seen = set()
    for t in range(T):
        k_ = int(key[t])
        if int(slot[t]) >= 0 and k_ in seen:
            keep[t] = False
        seen.add(k_)
    slot = torch.where(keep, slot, torch.full_like(slot, -1))
    table = torch.randperm(15, generator=torch.Generator().manual_seed(84)).to(torch.int32).view(3, 5).to(DEV)
    ang = torch.arange(400, device=DEV, dtype=torch.float64)[:, None] * \
        (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV, dtype=torch.float64) * 2 / hd))[None, :]
    cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    k0, v0 = _paged(15, n_kv, hd, torch.bfloat16, 85)
    qa, ka, va = qkv.clone(), k0.clone(), v0.clone()
    ops().rope_append(qa, cos, sin, pos, slot, table, ka, va, n_q, n_kv, hd, hd, 6, True)
    qb, kb, vb = qkv.clone(), k0.clone(), v0.clone()
    ops().rope_append_vec(qb, cos, sin, pos, slot, table, kb, vb, n_q, n_kv, hd, 6)
    torch.testing.assert_close(qb.float(), qa.float(), atol=0, rtol=2 ** -7)
    torch.testing.assert_close(kb.float(), ka.float(), atol=0, rtol=2 ** -7)
    assert torch.equal(vb, va)


# ---- random weights ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_random_fill_device_equals_host_bit_for_bit(dtype):
    """The same (seed, name) gives the same bits from the CUDA kernel, from the package's host
    version and from the tests' own scalar recipe; the offset of a piece is honoured."""
    import plain_random as pr
    from supersonic_b200.weights import random_fill
    for seed, name, mean, std, shape in ((2, "model.layers.31.mlp.down_proj.weight", 0.0, 0.02, (301, 257)),
                                         (9, "model.norm.weight", 1.0, 0.1, (4099,))):
        host = random_fill.fill_host(seed, name, shape, mean, std, dtype)
        dev = random_fill.fill_device(seed, name, shape, mean, std, DEV, dtype)
        assert torch.equal(dev.cpu(), host)
        if dtype == torch.bfloat16:
            got = dev.view(-1)[:50].view(torch.int16).cpu().tolist()
            assert [g & 0xFFFF for g in got] == [pr.value_bits(seed, name, i, mean, std) for i in range(50)]


def test_random_store_is_the_written_folder(tmp_path):
    """A folder written on the host and a store that makes its tensors on the device hold one model."""
    import tiny_configs
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import RandomWeightStore, WeightStore, write_model_folder
    cfg = config_from_dict(tiny_configs.B)
    write_model_folder(cfg, 5, str(tmp_path), std=0.05)
    folder = WeightStore.from_dir(str(tmp_path))
    made = RandomWeightStore(cfg, 5, device=DEV, std=0.05)
    for name in cfg.tensor_shapes():
        assert torch.equal(made.get(name).cpu(), folder.get(name)), name


def test_attention_decode_chunked_over_a_ragged_batch():
    """The persistent grid of the tensor-core kernel over sequences of 1 to 2,900 keys in one launch,
    more work items than blocks, several chunk sizes, a far key that stands out in a long sequence;
    and the cut of a sequence does not depend on the batch: alone or among the others, the same bits."""
    n_q, n_kv, hd = 8, 2, 128
    lens = [1, 2900, 64, 65, 700, 5, 1500, 129, 2047, 333, 1, 2048]
    B, n_pages = len(lens), 46
    g = torch.Generator(device=DEV).manual_seed(81)
    k, v = _paged(B * n_pages, n_kv, hd, torch.bfloat16, 82)
    table = torch.randperm(B * n_pages, generator=torch.Generator().manual_seed(83)).to(torch.int32).view(B, n_pages).to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    q = torch.randn(B, n_q * hd, device=DEV, generator=g).bfloat16()
    # sequence 1: key 37 (page 0) answers head 0's query far more loudly than any of the other 2,899
    k[int(table[1, 0]), 0, 37] = (q[1, :hd].float() * 4 / q[1, :hd].float().norm() * math.sqrt(hd)).bfloat16()
    scale = 1 / math.sqrt(hd)
    ref = _attention_reference(q, k, v, pos, slot, table, n_q, n_kv, hd, None, scale)
    assert (ref[1, :hd] - v[int(table[1, 0]), 0, 37].double()).abs().max() < 0.05      # the far key decides head 0
    for chunk, max_chunks in ((1, 46), (3, 16), (8, 6), (8, 3), (64, 1)):
        nf, nc = ops().attention_decode_chunked_scratch(B, n_q, n_kv, hd, max_chunks)
        scratch = torch.full((max(nf, 1),), float("nan"), device=DEV)
        counters = torch.zeros(nc, dtype=torch.int32, device=DEV)
        out = torch.full((B, n_q * hd), 5.0, dtype=torch.bfloat16, device=DEV)
        ops().attention_decode_chunked(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, None, scale, chunk,
                                       max_chunks, scratch, counters)
        torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)
        assert torch.all(counters == 0)
        for b in (1, 4, 10):                                             # alone: the same chunks, the same bits
            alone = torch.empty((1, n_q * hd), dtype=torch.bfloat16, device=DEV)
            ops().attention_decode_chunked(q[b:b + 1], k, v, pos[b:b + 1], slot[b:b + 1], table, alone, n_q, n_kv, hd,
                                           6, None, scale, chunk, max_chunks, scratch, counters)
            assert torch.equal(alone[0], out[b]), (chunk, b)


def test_kernels_with_scratch_stay_inside_it():
    """Guard words behind the scratch a kernel is told it may use: the chunked decode attention's partial
    results and counters, the split projection's partial tiles.  Nothing past the stated sizes changes."""
    n_q, n_kv, hd, B = 8, 2, 128, 5
    g = torch.Generator(device=DEV).manual_seed(91)
    k, v = _paged(B * 20, n_kv, hd, torch.bfloat16, 92)
    table = torch.randperm(B * 20, generator=torch.Generator().manual_seed(93)).to(torch.int32).view(B, 20).to(DEV)
    pos = torch.tensor([1279, 5, 640, 64, 1000], dtype=torch.int32, device=DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    q = torch.randn(B, n_q * hd, device=DEV, generator=g).bfloat16()
    out = torch.empty(B, n_q * hd, dtype=torch.bfloat16, device=DEV)
    chunk, max_chunks = 3, 7
    nf, nc = ops().attention_decode_chunked_scratch(B, n_q, n_kv, hd, max_chunks)
    scratch = torch.full((nf + 64,), 7.5, device=DEV)
    counters = torch.zeros(nc + 64, dtype=torch.int32, device=DEV)
    counters[nc:] = 12345
    ops().attention_decode_chunked(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, None, 1 / math.sqrt(hd), chunk,
                                   max_chunks, scratch, counters)
    torch.cuda.synchronize()
    assert torch.all(scratch[nf:] == 7.5) and torch.all(counters[nc:] == 12345) and torch.all(counters[:nc] == 0)
    ref = _attention_reference(q, k, v, pos, slot, table, n_q, n_kv, hd, None, 1 / math.sqrt(hd))
    torch.testing.assert_close(out.double(), ref, atol=2e-2, rtol=2e-2)
    rows, N, K, splits = 20, 1000, 4096, 5
    nf, nc = ops().gemv_tc_scratch(rows, N, splits)
    partials = torch.full((nf + 64,), 7.5, device=DEV)
    cnt = torch.zeros(nc + 64, dtype=torch.int32, device=DEV)
    cnt[nc:] = 12345
    x = torch.randn(rows, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    y = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
    ops().gemv_tc(x, w, y, splits=splits, partials=partials, counters=cnt)
    torch.cuda.synchronize()
    assert torch.all(partials[nf:] == 7.5) and torch.all(cnt[nc:] == 12345) and torch.all(cnt[:nc] == 0)
    torch.testing.assert_close(y.float(), x.float() @ w.float().T, atol=0.15, rtol=2e-2)
    ops().check_device_errors()
