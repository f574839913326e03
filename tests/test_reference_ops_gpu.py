"""The plain implementation's formulas against DeanoC/SuperSonic's own CUDA kernels.

``baseline/reference_kernels.py`` compiles the reference's bridge files unmodified for sm_100a
and binds their component launchers.  Each test feeds one of them bfloat16 inputs and compares
its output with the matching function of ``tests/plain_llama.py`` on the same (bfloat16-valued)
inputs: what differs is the reference's float32 arithmetic and its rounding of the result to
bfloat16 (2^-8 relative at most), so the bounds below are a few bfloat16 steps of the result.
Skipped, with the reason, where the libraries are not built (``python -m baseline.reference_kernels``).
"""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl
import tiny_configs
from baseline import reference_kernels as rk

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_STEP = 2.0 ** -8          # largest relative error of one rounding to bfloat16


@pytest.fixture(scope="module", autouse=True)
def reference_libraries():
    why = rk.available()
    if why:
        pytest.skip(f"the reference's kernels are not available: {why}")


def bf(a):
    """A float array rounded to bfloat16: (device tensor, the same values as float64)."""
    t = torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16).contiguous()
    return t, t.float().cpu().numpy().astype(np.float64)


def close(got, want, steps, floor=0.0):
    """|got - want| <= steps bfloat16 steps of |want| (+ floor), element-wise."""
    got = np.asarray(got, dtype=np.float64)
    err = np.abs(got - want)
    bound = steps * BF16_STEP * np.abs(want) + floor
    worst = np.argmax(err - bound)
    assert (err <= bound).all(), f"worst: got {got.flat[worst]} want {want.flat[worst]}"


CASES = [tiny_configs.A, tiny_configs.B, tiny_configs.E]


@pytest.mark.parametrize("cfg", CASES, ids=["A", "B", "E"])
def test_rms_norm(cfg):
    rng = np.random.default_rng(1)
    H = cfg["hidden_size"]
    x, x64 = bf(rng.normal(0, 2.0, (7, H)))
    w, w64 = bf(1.0 + rng.normal(0, 0.3, H))
    got = rk.rms_norm(x, w, cfg["rms_norm_eps"]).float().cpu().numpy()
    close(got, pl.rms_norm(x64, w64, cfg["rms_norm_eps"]), steps=1.01, floor=1e-6)


def test_rms_norm_small_values_feel_eps():
    """Rows so small that eps dominates the mean square: a wrong place for eps shows."""
    x, x64 = bf(np.full((2, 64), 1e-3))
    w, w64 = bf(np.ones(64))
    got = rk.rms_norm(x, w, 1e-5).float().cpu().numpy()
    close(got, pl.rms_norm(x64, w64, 1e-5), steps=1.01)
    assert abs(got[0, 0] - 1e-3 / math.sqrt(1e-6 + 1e-5)) < 2e-3


@pytest.mark.parametrize("cfg", CASES, ids=["A", "B", "E"])
def test_rope_pairs_and_positions(cfg):
    rng = np.random.default_rng(2)
    hd, nq = pl.head_dim_of(cfg), cfg["num_attention_heads"]
    first, T = 5, 9
    cos64, sin64 = pl.rope_tables(cfg, first + T)
    cos, cosr = bf(cos64)
    sin, sinr = bf(sin64)          # the reference keeps its tables in bfloat16 (llama31_engine.rs:147-157)
    x, x64 = bf(rng.normal(0, 1.0, (T, nq, hd)))
    got = rk.apply_rope_prefill(x.clone(), cos, sin, first_position=first).float().cpu().numpy()
    want = pl.apply_rope(x64, cosr[first:first + T], sinr[first:first + T])
    close(got, want, steps=1.01, floor=2e-3 * BF16_STEP)
    # the pairing is (i, i + hd/2): with the interleaved pairing (2i, 2i+1) the result differs widely
    inter = x64.copy()
    inter[..., 0::2] = x64[..., 0::2] * cosr[first:first + T, None, :] - x64[..., 1::2] * sinr[first:first + T, None, :]
    assert np.abs(got - inter).max() > 0.1


def test_swiglu():
    rng = np.random.default_rng(3)
    g, g64 = bf(rng.normal(0, 3.0, 1000))
    u, u64 = bf(rng.normal(0, 2.0, 1000))
    got = rk.swiglu_mul(g, u).float().cpu().numpy()
    close(got, g64 / (1.0 + np.exp(-g64)) * u64, steps=1.05, floor=1e-6)


@pytest.mark.parametrize("m,n,k", [(5, 33, 64), (40, 96, 100), (17, 448, 192)])
def test_tiled_matmul(m, n, k):
    rng = np.random.default_rng(4)
    a, a64 = bf(rng.normal(0, 1.0, (m, k)))
    w, w64 = bf(rng.normal(0, 0.1, (n, k)))
    got = rk.matmul_rhs_transposed(a, w).float().cpu().numpy()
    want = a64 @ w64.T
    close(got, want, steps=1.01, floor=2e-6 * math.sqrt(k))


def test_gemv_through_the_library():
    rng = np.random.default_rng(5)
    x, x64 = bf(rng.normal(0, 1.0, 192))
    w, w64 = bf(rng.normal(0, 0.1, (448, 192)))
    close(rk.gemv_bf16(x, w).float().cpu().numpy(), w64 @ x64, steps=1.01, floor=1e-5)


@pytest.mark.parametrize("cfg", CASES, ids=["A", "B", "E"])
def test_feed_forward_of_reference_kernels(cfg):
    """gate, up, SwiGLU, down, each a reference kernel with bfloat16 between them, against the plain
    feed-forward in float64: three roundings on the way."""
    rng = np.random.default_rng(6)
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    x, x64 = bf(rng.normal(0, 1.0, (6, H)))
    wg, wg64 = bf(rng.normal(0, 0.1, (I, H)))
    wu, wu64 = bf(rng.normal(0, 0.1, (I, H)))
    wd, wd64 = bf(rng.normal(0, 0.1, (H, I)))
    z = rk.swiglu_mul(rk.matmul_rhs_transposed(x, wg), rk.matmul_rhs_transposed(x, wu))
    got = rk.matmul_rhs_transposed(z, wd).float().cpu().numpy()
    want = pl.swiglu_ffn(x64, {"p.mlp.gate_proj.weight": wg64, "p.mlp.up_proj.weight": wu64,
                               "p.mlp.down_proj.weight": wd64}, "p")
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 4 * BF16_STEP * scale


def qkv(cfg, T, seed, spike=None):
    rng = np.random.default_rng(seed)
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], pl.head_dim_of(cfg)
    q = rng.normal(0, 1.0, (T, nq, hd))
    k = rng.normal(0, 1.0, (T, nkv, hd))
    v = rng.normal(0, 1.0, (T, nkv, hd))
    if spike is not None:          # one far key that every later query of head 0 finds
        k[spike] *= 0.1
        k[spike, 0, :] = 6.0 * q[-1, 0, :] / np.linalg.norm(q[-1, 0, :])
    return q, k, v


def heads_first(t):
    return t.permute(1, 0, 2).contiguous()[None]


@pytest.mark.parametrize("cfg", CASES, ids=["A", "B", "E"])
def test_prefill_attention(cfg):
    T = 70
    q64, k64, v64 = qkv(cfg, T, 7, spike=3)
    (q, qr), (k, kr), (v, vr) = bf(q64), bf(k64), bf(v64)
    scale = 1.0 / math.sqrt(pl.head_dim_of(cfg))
    got = rk.attention_prefill(heads_first(q), heads_first(k), heads_first(v), scale)[0]
    got = got.permute(1, 0, 2).cpu().numpy()
    want = pl.attention_scores(qr, kr, vr, scale)
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())     # float32 throughout, fast exp
    # group mapping: query head g reads kv head g // (nq / nkv)
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    if nkv > 1:
        swapped = pl.attention_scores(qr, kr[:, ::-1], vr[:, ::-1], scale)
        assert np.abs(got - swapped).max() > 0.05


@pytest.mark.parametrize("cfg", CASES, ids=["A", "B", "E"])
def test_prefill_attention_continues_a_cache(cfg):
    """The last rows of a sequence against all keys (seqlen_offset > 0) equal the whole pass's rows."""
    T, new = 50, 6
    q64, k64, v64 = qkv(cfg, T, 8)
    (q, qr), (k, kr), (v, vr) = bf(q64), bf(k64), bf(v64)
    scale = 1.0 / math.sqrt(pl.head_dim_of(cfg))
    got = rk.attention_prefill(heads_first(q[T - new:]), heads_first(k), heads_first(v), scale,
                               seqlen_offset=T - new)[0].permute(1, 0, 2).cpu().numpy()
    want = pl.attention_scores(qr, kr, vr, scale)[T - new:]
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("cfg", CASES, ids=["A", "B", "E"])
def test_decode_attention(cfg):
    """One query over a cache with spare room: the last row of the whole-sequence attention."""
    T, cap = 45, 64
    q64, k64, v64 = qkv(cfg, T, 9, spike=1)
    (q, qr), (k, kr), (v, vr) = bf(q64), bf(k64), bf(v64)
    nkv, hd = cfg["num_key_value_heads"], pl.head_dim_of(cfg)
    kc = torch.full((1, nkv, cap, hd), 7.0, dtype=torch.bfloat16, device=DEV)     # beyond kv_len: never read
    vc = torch.full((1, nkv, cap, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    kc[0, :, :T] = k.permute(1, 0, 2)
    vc[0, :, :T] = v.permute(1, 0, 2)
    scale = 1.0 / math.sqrt(hd)
    got = rk.attention_decode(q[T - 1][None].contiguous(), kc, vc, scale, kv_len=T)[0].float().cpu().numpy()
    want = pl.attention_scores(qr, kr, vr, scale)[T - 1]
    close(got, want, steps=1.05, floor=1e-4)


def test_head_argmax_takes_the_lowest_index_of_a_tie():
    rng = np.random.default_rng(10)
    H, V = 96, 384
    x, x64 = bf(rng.normal(0, 1.0, H))
    w64 = rng.normal(0, 0.1, (V, H))
    w64[300] = w64[41] = w64[200] = 0.3 * x64 / np.linalg.norm(x64)      # three equal, largest logits
    w, wr = bf(w64)
    for f32 in (False, True):
        got = rk.lm_head_argmax(x, w, f32_logits=f32)
        assert got == 41
    logits = wr @ x64
    assert pl.greedy_token(logits) == 41


def test_head_argmax_equals_plain_greedy_on_random_rows():
    rng = np.random.default_rng(11)
    H, V = 192, 777
    w, wr = bf(rng.normal(0, 0.1, (V, H)))
    for i in range(8):
        x, x64 = bf(rng.normal(0, 1.0, H))
        logits = wr @ x64
        top2 = np.sort(logits)[-2:]
        if top2[1] - top2[0] < 4 * BF16_STEP * abs(top2[1]):
            continue                       # a near-tie that rounding may decide either way
        assert rk.lm_head_argmax(x, w, f32_logits=True) == pl.greedy_token(logits)


def test_target_nll():
    rng = np.random.default_rng(12)
    logits, l64 = bf(rng.normal(0, 2.0, (5, 301)))
    targets = torch.tensor([0, 300, 17, 17, 128], dtype=torch.int32, device=DEV)
    got = rk.target_nll(logits, targets).cpu().numpy()
    m = l64.max(axis=1, keepdims=True)
    want = (m[:, 0] + np.log(np.exp(l64 - m).sum(axis=1))) - l64[np.arange(5), targets.cpu().numpy()]
    assert np.abs(got - want).max() < 1e-4


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_model_of_reference_kernels(name, model_folders):
    """A prompt through the reference's kernels alone (tests/reference_model.py) against the plain
    implementation: logits within the bfloat16 path's bound, and the same greedy tokens where the
    plain margin is not a near-tie."""
    import reference_model
    _, pc, pw = model_folders[name]
    rng = np.random.default_rng(13)
    tokens = rng.integers(0, pc["vocab_size"], 23).tolist()
    got = reference_model.forward(pc, pw, tokens, DEV)
    want = pl.forward(pc, pw, tokens)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 0.02 * scale
    for t in range(len(tokens)):
        top2 = np.sort(want[t])[-2:]
        if top2[1] - top2[0] > 0.04 * scale:
            assert int(np.argmax(got[t])) == pl.greedy_token(want[t])
