"""The plain implementation checked against properties that hold by definition, and
against the small golden file (CPU)."""
import importlib.util
import math
import os

import numpy as np

import plain_llama as pl
import tiny_configs


def test_rope_frequencies_llama3_by_hand():
    cfg = tiny_configs.B                      # theta 5e5, hd 32, factor 8, low 1, high 4, original 16
    inv = pl.rope_inv_freq(cfg)
    base = 1.0 / 500000.0 ** (np.arange(16) * 2 / 32)
    wavelen = 2 * math.pi / base
    c_inv = pl.rope_inv_freq(tiny_configs.C)  # theta 1e6, hd 48, factor 4, low 1, high 2, original 32
    c_base = 1.0 / 1000000.0 ** (np.arange(24) * 2 / 48)
    assert 2 * math.pi / c_base[0] < 16.0 and np.isclose(c_inv[0], c_base[0])     # short waves untouched
    assert np.isclose(c_inv[-1], c_base[-1] / 4.0)
    assert wavelen[-1] > 16.0 and np.isclose(inv[-1], base[-1] / 8.0)      # long waves divided by factor
    mid = [i for i in range(16) if 4.0 <= wavelen[i] <= 16.0]
    assert mid, "the configuration must exercise the blended band"
    for i in mid:
        s = (16.0 / wavelen[i] - 1.0) / 3.0
        assert np.isclose(inv[i], (1 - s) * base[i] / 8.0 + s * base[i])
    assert np.allclose(pl.rope_inv_freq(tiny_configs.A), 1.0 / 10000.0 ** (np.arange(8) * 2 / 16))


def test_rope_is_a_rotation_of_half_split_pairs():
    cos, sin = pl.rope_tables(tiny_configs.A, 9)
    x = np.random.default_rng(0).normal(size=(9, 3, 16))
    y = pl.apply_rope(x, cos, sin)
    assert np.allclose((x ** 2).sum(-1), (y ** 2).sum(-1))
    assert np.allclose(y[0], x[0])                                          # position 0: identity
    t, i = 5, 3
    c, s = cos[t, i], sin[t, i]
    assert np.isclose(y[t, 1, i], x[t, 1, i] * c - x[t, 1, i + 8] * s)
    assert np.isclose(y[t, 1, i + 8], x[t, 1, i] * s + x[t, 1, i + 8] * c)


def test_rms_norm_and_swiglu_by_hand():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(pl.rms_norm(x, np.array([2.0, 0.5]), 0.0), [[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]])
    w = {"p.mlp.gate_proj.weight": np.array([[1.0], [0.0]]), "p.mlp.up_proj.weight": np.array([[2.0], [5.0]]),
         "p.mlp.down_proj.weight": np.array([[1.0, 1.0]])}
    g = 0.7
    assert np.allclose(pl.swiglu_ffn(np.array([[g]]), w, "p"), g / (1 + math.exp(-g)) * 2 * g)


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(6, 4, 8)), rng.normal(size=(6, 2, 8)), rng.normal(size=(6, 2, 8))
    out = pl.attention_scores(q, k, v, 0.5)
    assert np.allclose(out[0, 0], v[0, 0]) and np.allclose(out[0, 3], v[0, 1])       # heads 0,1 -> kv 0; 2,3 -> kv 1
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = 9.0, -9.0
    assert np.allclose(pl.attention_scores(q, k2, v2, 0.5)[:4], out[:4])             # no look-ahead
    s = (q[5, 1] @ k[:, 0].T) * 0.5
    p = np.exp(s - s.max()); p /= p.sum()
    assert np.allclose(out[5, 1], p @ v[:, 0])
    w = pl.attention_scores(q, k, v, 0.5, window=2)
    s2 = s[4:]; p2 = np.exp(s2 - s2.max()); p2 /= p2.sum()
    assert np.allclose(w[5, 1], p2 @ v[4:, 0]) and np.allclose(w[0], out[0])


def test_logits_do_not_depend_on_later_tokens(model_folders):
    d, pc, pw = model_folders["A"]
    a = pl.forward(pc, pw, [1, 2, 3, 4, 5, 6])
    b = pl.forward(pc, pw, [1, 2, 3, 4, 200, 100])
    assert np.allclose(a[:4], b[:4]) and not np.allclose(a[4], b[4])
    assert a.shape == (6, pc["vocab_size"])


def test_sampling_distribution():
    logits = np.log(np.array([0.5, 0.2, 0.2, 0.1]))
    assert np.allclose(pl.sampling_distribution(logits, 1.0), [0.5, 0.2, 0.2, 0.1])
    assert np.allclose(pl.sampling_distribution(logits, 1.0, top_k=1), [1, 0, 0, 0])
    assert np.allclose(pl.sampling_distribution(logits, 1.0, top_k=2), [5 / 9, 2 / 9, 2 / 9, 0])   # ties kept
    assert np.allclose(pl.sampling_distribution(logits, 1.0, top_p=0.6), [5 / 9, 2 / 9, 2 / 9, 0])
    assert np.allclose(pl.sampling_distribution(logits, 1.0, top_p=0.5), [1, 0, 0, 0])
    p = pl.sampling_distribution(logits, 0.5)
    assert np.allclose(p, np.array([0.25, 0.04, 0.04, 0.01]) / 0.34)
    assert pl.greedy_token([1.0, 3.0, 3.0, 2.0]) == 1


def test_golden_file():
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    gold = np.load(os.path.join(here, "golden", "plain_logits.npz"))
    assert gold["tokens"].tolist() == mod.TOKENS
    assert np.allclose(mod.compute()[:, :48], gold["logits"], atol=1e-6)


def test_plain_against_the_reference_kernels_golden():
    """tests/golden/reference_kernels_logits.npz holds logits that DeanoC/SuperSonic's own CUDA
    kernels (compiled unmodified, chained as its prompt engine chains them: tests/reference_model.py)
    produced on a B200 for two tiny random models.  The plain implementation must agree within the
    bound of a path that rounds to bfloat16 after every operation (2 % of the largest logit)."""
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_reference_golden",
                                                  os.path.join(here, "golden", "make_reference_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    gold = np.load(os.path.join(here, "golden", "reference_kernels_logits.npz"))
    for name, toks in mod.TOKENS.items():
        assert gold[f"tokens_{name}"].tolist() == toks
        pc, pw = mod.model(name)
        want = pl.forward(pc, pw, toks)
        got = gold[f"logits_{name}"]
        assert np.abs(got - want[:, :64]).max() <= 0.02 * np.abs(want).max()
        clear = [t for t in range(len(toks)) if np.diff(np.sort(want[t, :64])[-2:])[0] > 0.04 * np.abs(want).max()]
        assert len(clear) >= len(toks) // 2
        for t in clear:           # the same best token among the stored columns wherever the margin is clear
            assert int(np.argmax(got[t])) == int(np.argmax(want[t, :64]))


def _cpp_plain(tmp_path):
    """Compile tests/plain_cpp/plain_llama.cpp once; None if there is no C++ compiler."""
    import shutil
    import subprocess
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        return None
    exe = str(tmp_path / "plain_llama")
    src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_cpp", "plain_llama.cpp")
    subprocess.run([cxx, "-O2", "-std=c++17", "-o", exe, src], check=True)
    return exe


def test_two_plain_statements_agree(model_folders, tmp_path):
    """The NumPy statement and the C++ one (tests/plain_cpp/plain_llama.cpp), written separately from
    the reference's formulas, give the same logits on two tiny models that differ in every option:
    tied and untied heads, with and without llama3 frequency scaling, positions past the scaling's
    original context."""
    import struct
    import subprocess
    import pytest
    exe = _cpp_plain(tmp_path)
    if exe is None:
        pytest.skip("no C++ compiler")
    for name, n_tokens in (("A", 21), ("B", 40)):
        _, pc, pw = model_folders[name]
        tokens = np.random.default_rng(5).integers(0, pc["vocab_size"], n_tokens).tolist()
        sc = pc.get("rope_scaling")
        nq = pc["num_attention_heads"]
        hdr = [pc["vocab_size"], pc["hidden_size"], pc["intermediate_size"], pc["num_hidden_layers"], nq,
               pc.get("num_key_value_heads") or nq, pl.head_dim_of(pc), int(bool(pc.get("tie_word_embeddings"))),
               n_tokens, int(bool(sc))]
        par = [pc["rms_norm_eps"], pc.get("rope_theta", 10000.0)] + (
            [sc["factor"], sc["low_freq_factor"], sc["high_freq_factor"], sc["original_max_position_embeddings"]]
            if sc else [1.0, 1.0, 1.0, 1.0])
        order = ["model.embed_tokens.weight"]
        for n in range(pc["num_hidden_layers"]):
            p = f"model.layers.{n}"
            order += [f"{p}.input_layernorm.weight", f"{p}.self_attn.q_proj.weight", f"{p}.self_attn.k_proj.weight",
                      f"{p}.self_attn.v_proj.weight", f"{p}.self_attn.o_proj.weight", f"{p}.post_attention_layernorm.weight",
                      f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight", f"{p}.mlp.down_proj.weight"]
        order.append("model.norm.weight")
        if not pc.get("tie_word_embeddings"):
            order.append("lm_head.weight")
        src, dst = tmp_path / f"{name}.in", tmp_path / f"{name}.out"
        with open(src, "wb") as f:
            f.write(struct.pack("<10q", *hdr))
            f.write(struct.pack("<6d", *[float(x) for x in par]))
            f.write(np.asarray(tokens, dtype="<i8").tobytes())
            for key in order:
                f.write(np.ascontiguousarray(pw[key], dtype="<f8").tobytes())
        subprocess.run([exe, str(src), str(dst)], check=True)
        got = np.fromfile(dst, dtype="<f8").reshape(n_tokens, pc["vocab_size"])
        want = pl.forward(pc, pw, tokens)
        assert np.abs(got - want).max() < 1e-9, name
