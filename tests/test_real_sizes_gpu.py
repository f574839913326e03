"""Llama-3.1-8B sizes (width 4096, 32/8 heads of 128, feed-forward 14336, a vocabulary of 128256)
with random weights against the plain implementation: the shapes the benchmark times, checked for
what they compute; one layer in detail, and all 32 layers in every batching.  A prompt of 140 tokens in one step (the
tcgen05 GEMM and attention in bfloat16), then tokens one by one (the decode projections and
attention), in float32 and in bfloat16.  Logits are compared on 2,000 vocabulary rows, so that
the plain side never multiplies by the whole head."""
import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol_abs,tol_rel", [("float32", 1e-4, 0.0), ("bfloat16", 0.0, 2e-2)])
def test_one_layer_at_8b_sizes(dtype, tol_abs, tol_rel):
    from supersonic_b200.config import preset_config
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import RandomWeightStore
    cfg = preset_config("llama3.1-8b", num_hidden_layers=1)
    store = RandomWeightStore(cfg, seed=5, device="cuda:0", std=0.02, norm_jitter=0.1)
    model = Model.from_config(cfg, store, dtype=dtype, device="cuda:0", max_tokens=512)
    pc = cfg.to_dict()
    rng = np.random.default_rng(13)
    toks = rng.integers(0, cfg.vocab_size, 144).tolist()
    rows = np.sort(rng.choice(cfg.vocab_size, 2000, replace=False))

    # the plain side: the prompt's embedding rows, the layer, the final norm, 2,000 rows of the head
    def host(name, index=None):
        t = store.get(name)
        return (t if index is None else t[torch.as_tensor(index, device=t.device)]).double().cpu().numpy()
    pw = {n: host(n) for n in store.names() if n.startswith("model.layers.0.")}
    cos, sin = pl.rope_tables(pc, len(toks))
    h = pl.block(host("model.embed_tokens.weight", toks), pw, 0, pc, cos, sin)
    ref = pl.rms_norm(h, host("model.norm.weight"), pc["rms_norm_eps"]) @ host("lm_head.weight", rows).T
    del pw
    tol = tol_abs + tol_rel * np.abs(ref).max()

    s = model.open_sequence()
    want = [0, 63, 64, 127, 139]
    got = model.step([StepEntry(s, toks[:140], want)])[:, torch.as_tensor(rows, device="cuda:0")]
    assert np.abs(got.double().cpu().numpy() - ref[want]).max() < tol
    for p in range(140, 144):
        got = model.step([StepEntry(s, [toks[p]], [0])])[:, torch.as_tensor(rows, device="cuda:0")]
        assert np.abs(got.double().cpu().numpy()[0] - ref[p]).max() < tol, p
    model.check_errors()


def test_a_batch_of_twenty_at_8b_sizes():
    """bfloat16, twenty sequences of unequal lengths: their prompts in one step, then two steps of
    twenty rows (the decode projections with 32 batch columns, attention over unequal contexts)."""
    from supersonic_b200.config import preset_config
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import RandomWeightStore
    cfg = preset_config("llama3.1-8b", num_hidden_layers=1)
    store = RandomWeightStore(cfg, seed=6, device="cuda:0", std=0.02, norm_jitter=0.1)
    model = Model.from_config(cfg, store, dtype="bfloat16", device="cuda:0", max_tokens=4096)
    pc = cfg.to_dict()
    rng = np.random.default_rng(14)
    seqs = [rng.integers(0, cfg.vocab_size, int(n)).tolist() for n in rng.integers(5, 70, 20)]
    rows = np.sort(rng.choice(cfg.vocab_size, 1500, replace=False))
    dev_rows = torch.as_tensor(rows, device="cuda:0")

    def host(name, index=None):
        t = store.get(name)
        return (t if index is None else t[torch.as_tensor(index, device=t.device)]).double().cpu().numpy()
    pw = {n: host(n) for n in store.names() if n.startswith("model.layers.0.")}
    norm_w, head = host("model.norm.weight"), host("lm_head.weight", rows)
    refs = []
    for t in seqs:
        cos, sin = pl.rope_tables(pc, len(t))
        h = pl.block(host("model.embed_tokens.weight", t), pw, 0, pc, cos, sin)
        refs.append(pl.rms_norm(h, norm_w, pc["rms_norm_eps"]) @ head.T)
    del pw
    tol = 2e-2 * max(np.abs(r).max() for r in refs)

    slots = [model.open_sequence() for _ in seqs]
    cut = [len(t) - 2 for t in seqs]
    got = model.step([StepEntry(s, t[:c], [c - 1]) for s, t, c in zip(slots, seqs, cut)])[:, dev_rows]
    got = got.double().cpu().numpy()
    for i, (r, c) in enumerate(zip(refs, cut)):
        assert np.abs(got[i] - r[c - 1]).max() < tol, i
    for step in range(2):
        got = model.step([StepEntry(s, [t[c + step]], [0]) for s, t, c in zip(slots, seqs, cut)])[:, dev_rows]
        got = got.double().cpu().numpy()
        for i, (r, c) in enumerate(zip(refs, cut)):
            assert np.abs(got[i] - r[c + step]).max() < tol, (step, i)
    model.check_errors()


def test_the_whole_model_at_8b_sizes_in_every_batching():
    """All 32 layers at Llama-3.1-8B sizes: the depth and width the benchmark times.  The float32
    path against the plain implementation, streamed layer by layer so that the host holds one layer
    in float64 at a time: a 24-token prompt whole; 16 tokens in one step and the last 8 one by one;
    three unequal prompts as one batch and two decode steps of it.  Every logit compared is within
    1e-4 on 2,000 vocabulary rows.  Then the bfloat16 path at the same places against that float32,
    within the rounding noise of 32 layers."""
    from supersonic_b200.config import preset_config
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import RandomWeightStore
    cfg = preset_config("llama3.1-8b")
    L = cfg.num_hidden_layers
    store = RandomWeightStore(cfg, seed=7, device="cuda:0", std=0.02, norm_jitter=0.1)
    pc = cfg.to_dict()
    rng = np.random.default_rng(15)
    seqs = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (24, 7, 15)]
    rows = np.sort(rng.choice(cfg.vocab_size, 2000, replace=False))
    dev_rows = torch.as_tensor(rows, device="cuda:0")

    def host(name, index=None):
        t = store.get(name)
        return (t if index is None else t[torch.as_tensor(index, device=t.device)]).double().cpu().numpy()

    hs = [host("model.embed_tokens.weight", t) for t in seqs]
    tables = [pl.rope_tables(pc, len(t)) for t in seqs]
    for n in range(L):
        pw = {name: host(name) for name in store.names() if name.startswith(f"model.layers.{n}.")}
        hs = [pl.block(h, pw, n, pc, cos, sin) for h, (cos, sin) in zip(hs, tables)]
        del pw
    norm_w, head = host("model.norm.weight"), host("lm_head.weight", rows)
    refs = [pl.rms_norm(h, norm_w, pc["rms_norm_eps"]) @ head.T for h in hs]
    scale = max(np.abs(r).max() for r in refs)

    def run(dtype):
        """{(sequence, position, schedule): logits row}"""
        m = Model.from_config(cfg, store, dtype=dtype, device="cuda:0", max_tokens=512)
        out = {}
        take = lambda t: t[:, dev_rows].double().cpu().numpy()
        a = seqs[0]
        s = m.open_sequence()                                   # whole
        for p, row in enumerate(take(m.step([StepEntry(s, a, range(24))]))):
            out[(0, p, "whole")] = row
        m.close_sequence(s)
        s = m.open_sequence()                                   # 16 at once, 8 one by one (in the slot just freed)
        out[(0, 15, "cut")] = take(m.step([StepEntry(s, a[:16], [15])]))[0]
        for p in range(16, 24):
            out[(0, p, "cut")] = take(m.step([StepEntry(s, [a[p]], [0])]))[0]
        m.close_sequence(s)
        slots = [m.open_sequence() for _ in seqs]               # three unequal prompts together
        cut = [len(t) - 2 for t in seqs]
        got = take(m.step([StepEntry(sl, t[:c], [c - 1]) for sl, t, c in zip(slots, seqs, cut)]))
        for i, c in enumerate(cut):
            out[(i, c - 1, "batch")] = got[i]
        for step in range(2):
            got = take(m.step([StepEntry(sl, [t[c + step]], [0]) for sl, t, c in zip(slots, seqs, cut)]))
            for i, c in enumerate(cut):
                out[(i, c + step, "batch")] = got[i]
        m.check_errors()
        m.cache.check()
        del m
        torch.cuda.empty_cache()
        return out

    f32 = run("float32")
    assert len(f32) == 24 + 9 + 9
    for (i, p, how), row in f32.items():
        err = np.abs(row - refs[i][p]).max()
        assert err <= 1e-4, f"float32, sequence {i}, position {p}, {how}: {err:.2e}"
    # bfloat16 at this depth: about six roundings of the activations a layer leave a noise of
    # sqrt(6 * 32) * 2^-9 = 2.7 % of a row's spread; a fault (a wrong page, position or head) leaves
    # about 100 %.  Per row: the error's root mean square against the spread of the float32 logits.
    bf16 = run("bfloat16")
    for key, row in bf16.items():
        rel = np.sqrt(np.mean((row - f32[key]) ** 2)) / f32[key].std()
        assert rel < 0.05, f"bfloat16 {key}: {rel:.3f}"
        assert np.abs(row - f32[key]).max() <= 0.05 * scale, f"bfloat16 {key}"
