"""Generation on the GPU through the Python entry point and the command line: greedy
tokens against the plain implementation, long decoding, the first tokens of a sequence,
stop tokens, sampling that does not depend on the batch."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as pl
import replay_helpers as rh

pytestmark = pytest.mark.gpu


def margin_ok(pc, pw, tokens, tol):
    """True if the plain top two logits at the last position differ by more than ``tol``."""
    top2 = np.sort(pl.forward(pc, pw, tokens)[-1])[-2:]
    return top2[1] - top2[0] > tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_matches_plain(model_folders, name, dtype):
    import supersonic_b200
    d, pc, pw = model_folders[name]
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, pc["vocab_size"], n).tolist() for n in (5, 11, 17, 1, 66)]
    eng = supersonic_b200.load(d, dtype=dtype, context_size=128, batch_size=3)
    got = eng.generate(prompts, max_new_tokens=8, ignore_eos=True, batch_size=3)
    tol = 1e-4 if dtype == "float32" else 4e-2
    for p, g in zip(prompts, got):
        assert len(g) == 8
        for i in range(8):
            # every token against the plain logits of the engine's own prefix: a token that is not
            # the plain best must be within a near-tie of it; the tokens after it are still checked
            logits = pl.forward(pc, pw, p + g[:i])[-1]
            best = pl.greedy_token(logits)
            assert g[i] == best or logits[best] - logits[g[i]] <= tol, (name, dtype, p, i, g)
    assert eng.model.cache.slots.n_held == 0
    eng.model.cache.check()


def test_stop_tokens_end_sequences_early(model_folders):
    import supersonic_b200
    d, pc, pw = model_folders["A"]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, 256, n).tolist() for n in (9, 3, 30, 12)]
    free = [pl.greedy_generate(pc, pw, p, 12) for p in prompts]
    stops = sorted({f[2] for f in free[:2]} | {free[2][7]})          # ends sequences at different steps
    eng = supersonic_b200.load(d, dtype="float32", context_size=128, batch_size=4)
    res = eng.generate_detailed(prompts, max_new_tokens=12, stop_token_ids=stops, batch_size=4)
    for p, r in zip(prompts, res):
        want = pl.greedy_generate(pc, pw, p, 12, stop_ids=stops)
        assert r.tokens == want
        assert r.finish_reason == ("stop" if want[-1] in stops else "length")
    assert len({len(r.tokens) for r in res}) > 1
    # config.json's eos_token_id (7 for this model) is the default stop set
    assert eng.model.spec.stop_token_ids == [7]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_logits(model_folders, dtype):
    """300 decoded tokens (several pages) with teacher forcing through the step function."""
    from supersonic_b200.engine import Model, StepEntry
    d, pc, pw = model_folders["C"]
    toks = np.random.default_rng(7).integers(0, pc["vocab_size"], 330).tolist()
    ref = pl.forward(pc, pw, toks)
    m = Model.from_dir(d, dtype=dtype, max_tokens=384)
    s = m.open_sequence()
    m.step([StepEntry(s, toks[:30], [])])
    rows = [m.step([StepEntry(s, [toks[p]], [0])]) for p in range(30, 330)]
    got = torch.cat(rows).double().cpu().numpy()
    err = np.abs(got - ref[30:]).max(axis=1)
    tol = 2e-5 if dtype == "float32" else 2e-2 * np.abs(ref).max()
    assert err.max() < tol, f"first bad position {30 + int(np.argmax(err > tol))}"


@pytest.mark.parametrize("name", ["D", "E"])
def test_long_prompt_then_decoding_over_many_pages(model_folders, name):
    """bfloat16 with head sizes 64 and 128: a prompt of 1,100 tokens in one step (attention tiles
    with many blocks of keys), a second piece of 300 tokens that continues the cached prefix, then
    tokens one by one over 22 pages (decode attention with several splits), beside a short
    sequence that shares the batch."""
    from supersonic_b200.engine import Model, StepEntry
    d, pc, pw = model_folders[name]
    rng = np.random.default_rng(12)
    long_toks = rng.integers(0, pc["vocab_size"], 1430).tolist()
    short = rng.integers(0, pc["vocab_size"], 40).tolist()
    ref_long, ref_short = pl.forward(pc, pw, long_toks), pl.forward(pc, pw, short)
    tol = 2e-2 * max(np.abs(ref_long).max(), np.abs(ref_short).max())
    m = Model.from_dir(d, dtype="bfloat16", max_tokens=2048)
    a, b = m.open_sequence(), m.open_sequence()
    want = [0, 127, 128, 640, 1099]
    got = m.step([StepEntry(a, long_toks[:1100], want)]).double().cpu().numpy()
    assert np.abs(got - ref_long[want]).max() < tol
    want2 = [0, 150, 299]
    got = m.step([StepEntry(a, long_toks[1100:1400], want2), StepEntry(b, short[:10], [9])]).double().cpu().numpy()
    assert np.abs(got[:3] - ref_long[[1100 + w for w in want2]]).max() < tol
    assert np.abs(got[3] - ref_short[9]).max() < tol
    for i in range(30):
        got = m.step([StepEntry(a, [long_toks[1400 + i]], [0]), StepEntry(b, [short[10 + i]], [0])]).double().cpu().numpy()
        assert np.abs(got[0] - ref_long[1400 + i]).max() < tol, i
        assert np.abs(got[1] - ref_short[10 + i]).max() < tol, i
    m.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(model_folders, dtype):
    """Positions 0, 1, 2 decoded one by one from an empty slot, for two sequences at once."""
    from supersonic_b200.engine import Model, StepEntry
    d, pc, pw = model_folders["B"]
    a, b = [11, 200, 3, 77], [380, 0, 0, 5]
    ra, rb = pl.forward(pc, pw, a), pl.forward(pc, pw, b)
    m = Model.from_dir(d, dtype=dtype, max_tokens=128)
    sa, sb = m.open_sequence(), m.open_sequence()
    tol = 2e-5 if dtype == "float32" else 2e-2 * max(np.abs(ra).max(), np.abs(rb).max())
    for p in range(4):
        lg = m.step([StepEntry(sa, [a[p]], [0]), StepEntry(sb, [b[p]], [0])]).double().cpu().numpy()
        assert np.abs(lg[0] - ra[p]).max() < tol and np.abs(lg[1] - rb[p]).max() < tol, p


def test_sampling_does_not_depend_on_the_batch(model_folders):
    import supersonic_b200
    d, pc, pw = model_folders["B"]
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, 384, n).tolist() for n in (1, 7, 19, 40)]
    eng = supersonic_b200.load(d, dtype="float32", context_size=128, batch_size=4)
    kw = dict(max_new_tokens=12, temperature=0.7, sampling_seed=1234, ignore_eos=True)
    together = eng.generate(prompts, batch_size=4, **kw)
    assert together == eng.generate(prompts, batch_size=4, **kw)          # the seed decides
    pairs = eng.generate(prompts, batch_size=2, **kw)
    assert pairs == together                                              # the batch does not
    assert eng.generate(prompts, batch_size=4, **{**kw, "sampling_seed": 99}) != together
    assert eng.generate(prompts, batch_size=4, **{**kw, "top_k": 1}) == \
        eng.generate(prompts, batch_size=4, max_new_tokens=12, ignore_eos=True)   # top_k 1 is greedy
    # every sampled token is one the plain distribution allows under top-k
    limited = eng.generate(prompts[:2], batch_size=2, **{**kw, "top_k": 5})
    for p, g in zip(prompts[:2], limited):
        seq = list(p)
        for t in g:
            probs = pl.sampling_distribution(pl.forward(pc, pw, seq)[-1], 0.7, top_k=5)
            assert probs[t] > 0
            seq.append(t)


def test_command_line(model_folders):
    d, pc, pw = model_folders["A"]
    prompt = [5, 9, 100, 42]
    want = pl.greedy_generate(pc, pw, prompt, 6)
    cmd = [sys.executable, os.path.join(rh.ROOT, "bin", "supersonic"), "--model-dir", d, "--prompt-ids",
           ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", "float32", "--ignore-eos",
           "--emit-generated-json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("[tokens] ")][0]
    assert [int(t) for t in line.split()[1:]] == want
    assert "[generated_json]" in proc.stdout and "[result] prompt_tokens=4 generated_tokens=6" in proc.stderr


def test_no_cpu_path():
    from supersonic_b200.engine import Model
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import random_store
    import tiny_configs
    c = config_from_dict(tiny_configs.A)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Model.from_config(c, random_store(c, 0), device="cpu")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_widths_the_fast_kernels_refuse_still_give_the_right_logits(tmp_path, dtype):
    """A width and a feed-forward width that are no multiple of 8, an odd vocabulary, three kv
    heads: the vector kernels do not take these, the plain ones must, with the same results."""
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import write_model_folder
    cfg = dict(architectures=["LlamaForCausalLM"], vocab_size=301, hidden_size=68, intermediate_size=100,
               num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3, head_dim=16,
               max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True)
    d = write_model_folder(config_from_dict(cfg), 9, str(tmp_path / "m"), std=0.1)
    pc, pw = pl.read_model_folder(d)
    toks = np.random.default_rng(9).integers(0, 301, 100).tolist()
    ref = pl.forward(pc, pw, toks)
    m = Model.from_dir(d, dtype=dtype, max_tokens=128)
    s = m.open_sequence()
    got = [m.step([StepEntry(s, toks[:90], range(90))])]
    got += [m.step([StepEntry(s, [toks[p]], [0])]) for p in range(90, 100)]
    got = torch.cat(got).double().cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 2e-2 * np.abs(ref).max()
    assert np.abs(got - ref).max() < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,budget", [("B", 7), ("D", 100), ("E", 129)])
def test_a_step_over_its_token_budget_runs_in_chunks_with_the_same_logits(model_folders, name, budget, dtype):
    """Three prompts of unequal lengths in one step that the model cuts into chunks (a prompt ends
    inside a chunk, a prompt spans three chunks, a chunk holds one token of a prompt), then decoding:
    the wanted logits come back in the order of the entries and of their places, and equal the
    plain implementation's."""
    from supersonic_b200.engine import Model, StepEntry
    d, pc, pw = model_folders[name]
    rng = np.random.default_rng(21)
    lens = [budget + 1, 3, 2 * budget + 5] if name != "B" else [8, 3, 19]
    seqs = [rng.integers(0, pc["vocab_size"], n + 2).tolist() for n in lens]
    refs = [pl.forward(pc, pw, s) for s in seqs]
    tol = 2e-5 if dtype == "float32" else 2e-2 * max(np.abs(r).max() for r in refs)
    m = Model.from_dir(d, dtype=dtype, max_tokens=1024, step_token_budget=budget)
    slots = [m.open_sequence() for _ in seqs]
    wants = [[0, n - 1] for n in lens]
    wants[2] = [0, budget - 1, budget, lens[2] - 1]
    got = m.step([StepEntry(s, q[:n], w) for s, q, n, w in zip(slots, seqs, lens, wants)]).double().cpu().numpy()
    want_rows = np.concatenate([r[w] for r, w in zip(refs, wants)])
    assert got.shape == want_rows.shape
    assert np.abs(got - want_rows).max() < tol
    assert [m.cache.length(s) for s in slots] == lens
    for t in range(2):
        got = m.step([StepEntry(s, [q[n + t]], [0]) for s, q, n in zip(slots, seqs, lens)]).double().cpu().numpy()
        assert np.abs(got - np.stack([r[n + t] for r, n in zip(refs, lens)])).max() < tol
    for s in slots:
        m.close_sequence(s)
    m.cache.check()
    # a step that does not fit the cache runs nothing
    s0 = m.open_sequence()
    with pytest.raises(Exception):
        m.step([StepEntry(s0, [1] * 2000, [])])
    assert m.cache.length(s0) == 0


@pytest.mark.parametrize("head_dim,tokens", [(128, 20000), (64, 12000)])
def test_a_far_context_in_bfloat16_stays_on_the_float32_path(head_dim, tokens):
    """Hundreds of pages: a prompt of ``tokens`` tokens cut into chunks of 8,192 (the tcgen05 attention
    over a long cached prefix), then 24 tokens one by one beside a short sequence (decode attention
    in many chunks, lengths that differ by a factor of 60).  The plain implementation would take
    minutes here, so the oracle is the engine's own float32 path, which the other tests pin to it:
    every wanted row of bfloat16 logits lies within 5 % (root mean square, relative) of float32's."""
    from supersonic_b200.config import preset_config
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import RandomWeightStore
    cfg = preset_config("llama3.1-8b", num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=head_dim, intermediate_size=512, vocab_size=1000,
                        eos_token_id=1, bos_token_id=0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (tokens + 24,), generator=g).tolist()
    short = torch.randint(0, cfg.vocab_size, (224,), generator=g).tolist()
    want = [0, 8191, 8192, tokens - 1]
    rows = {}
    for dtype in ("bfloat16", "float32"):
        store = RandomWeightStore(cfg, seed=7, device="cuda:0", std=0.05, norm_jitter=0.1)
        m = Model.from_config(cfg, store, dtype=dtype, device="cuda:0", max_tokens=tokens + 1024,
                              max_seq_tokens=tokens + 64, step_token_budget=8192)
        a, b = m.open_sequence(), m.open_sequence()
        got = [m.step([StepEntry(a, toks[:tokens], want), StepEntry(b, short[:200], [199])]).float().cpu()]
        for i in range(24):
            got.append(m.step([StepEntry(a, [toks[tokens + i]], [0]), StepEntry(b, [short[200 + i]], [0])]).float().cpu())
        rows[dtype] = torch.cat(got)
        m.cache.check()
        del m, store
    ref, got = rows["float32"], rows["bfloat16"]
    rel = (got - ref).pow(2).mean(dim=1).sqrt() / ref.pow(2).mean(dim=1).sqrt()
    assert float(rel.max()) < 0.05, rel


def test_a_model_the_device_cannot_hold_is_refused_before_anything_is_loaded(model_folders):
    from supersonic_b200.engine import Model
    from supersonic_b200.engine.preflight import MemoryPreflightError
    d, pc, pw = model_folders["A"]
    torch.cuda.empty_cache()
    free_before = torch.cuda.mem_get_info()[0]
    with pytest.raises(MemoryPreflightError, match=r"\[vram\] estimated=.*kv_cache=.*do not fit"):
        Model.from_dir(d, dtype="float32", max_tokens=1 << 34, max_seq_tokens=256, max_slots=4)
    torch.cuda.empty_cache()
    assert torch.cuda.mem_get_info()[0] >= free_before - (64 << 20)      # nothing of it was allocated
    m = Model.from_dir(d, dtype="float32", max_tokens=256)                # and the device is as usable as before
    est = m.memory_estimate
    assert est.cache == m.cache.bytes_held() and est.weights > 0 and est.workspace > 0


@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", True), ("bfloat16", False)])
def test_a_position_limit_that_is_no_multiple_of_the_page_size(tmp_path, dtype, graphs):
    """max_position_embeddings = 100: the cache's pages would hold 128 tokens, the rotary tables have
    100 rows.  Decoding runs up to the limit with the right logits and is refused beyond it, with
    captured graphs (which cannot see positions on the host) and without."""
    import tiny_configs
    from supersonic_b200.cache import CacheFull
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import write_model_folder
    cfg = dict(tiny_configs.D, max_position_embeddings=100)
    write_model_folder(config_from_dict(cfg), 3, str(tmp_path), std=0.07)
    pc, pw = pl.read_model_folder(str(tmp_path))
    toks = np.random.default_rng(21).integers(0, pc["vocab_size"], 101).tolist()
    ref = pl.forward(pc, pw, toks[:100])
    m = Model.from_dir(str(tmp_path), dtype=dtype, max_tokens=256, use_graphs=graphs)
    assert m.use_graphs == graphs and m.cache.max_seq_tokens == 100
    s = m.open_sequence()
    m.step([StepEntry(s, toks[:90], [])])
    rows = [m.step([StepEntry(s, [toks[p]], [0])]) for p in range(90, 100)]
    got = torch.cat(rows).double().cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 2e-2 * np.abs(ref).max()
    assert np.abs(got - ref[90:]).max() < tol
    with pytest.raises((CacheFull, ValueError)):
        m.step([StepEntry(s, [toks[100]], [0])])
    assert m.cache.length(s) == 100
    m.cache.check()
    # the generation loop refuses a request that would pass the limit before it runs anything
    import supersonic_b200
    eng = supersonic_b200.load(str(tmp_path), dtype=dtype, batch_size=1)
    assert len(eng.generate([toks[:92]], max_new_tokens=8, ignore_eos=True)[0]) == 8
    with pytest.raises(ValueError, match="exceed"):
        eng.generate([toks[:95]], max_new_tokens=8, ignore_eos=True)


def _run_cli(*args):
    cmd = [sys.executable, os.path.join(rh.ROOT, "bin", "supersonic")] + [str(a) for a in args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600)


def _preset_plain(name, seed, tmp_path):
    """The plain side of ``--preset NAME --random-seed SEED``: the same generator writes the folder."""
    from supersonic_b200.config import preset_config
    from supersonic_b200.weights import write_model_folder
    write_model_folder(preset_config(name), seed, str(tmp_path), std=0.02, norm_jitter=0.0)
    return pl.read_model_folder(str(tmp_path))


def test_command_line_with_a_preset_a_prompt_file_and_stop_ids(tmp_path):
    """``--preset tiny-b --random-seed 5`` makes its weights on the device; a folder written on the host
    from the same seed is the same model, so the plain implementation can check the tokens.  Three
    prompts from a file at batch size 2: two batches, and [prefill] counts all three prompts."""
    pc, pw = _preset_plain("tiny-b", 5, tmp_path / "m")
    rng = np.random.default_rng(51)
    prompts = [rng.integers(0, pc["vocab_size"], n).tolist() for n in (6, 13, 4)]
    free = [pl.greedy_generate(pc, pw, p, 7) for p in prompts]
    stop = free[1][3]
    f = tmp_path / "prompts.txt"
    f.write_text("# three prompts\n" + "\n".join(", ".join(map(str, p)) for p in prompts[:2]) + "\n\n"
                 + " ".join(map(str, prompts[2])) + "  # spaces work too\n")
    proc = _run_cli("--preset", "tiny-b", "--random-seed", 5, "--prompt-file", f, "--max-new-tokens", 7,
                    "--dtype", "float32", "--stop-ids", stop, "--batch-size", 2, "--emit-stage-timings")
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = [[int(t) for t in l.split()[1:]] for l in proc.stdout.splitlines() if l.startswith("[tokens] ")]
    assert got == [pl.greedy_generate(pc, pw, p, 7, stop_ids=[stop]) for p in prompts]
    assert got[1][-1] == stop and len(got[1]) <= 4          # the second prompt ends at the stop token
    assert "[prefill] 23 tokens in" in proc.stderr and "(2 batches)" in proc.stderr
    assert "[vram] estimated=" in proc.stderr
    stage = [l for l in proc.stderr.splitlines() if l.startswith("[stage] decode")][0]
    fields = dict(kv.split("=") for kv in stage.split()[2:])
    assert float(fields["full_attn_proj"]) > 0 and float(fields["full_attn_core"]) > 0 and float(fields["mlp"]) > 0
    assert float(fields["rms_norm"]) > 0 and float(fields["lm_head"]) > 0 and float(fields["sampling"]) > 0
    assert abs(float(fields["full_attn"]) - float(fields["full_attn_proj"]) - float(fields["full_attn_core"])) < 0.2


def test_command_line_refusals():
    assert _run_cli("--prompt-ids", "1,2").returncode == 2                         # no model
    assert _run_cli("--preset", "no-such", "--prompt-ids", "1").returncode == 2
    assert _run_cli("--preset", "tiny-a", "--prompt-ids", "1,x").returncode == 2
    assert _run_cli("--preset", "tiny-a", "--prompt-ids", "1,2,3", "--context-size", 4).returncode == 2
    out = _run_cli("--list-presets")
    assert out.returncode == 0 and "llama3.1-8b" in out.stdout and "tiny-a" in out.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode_step", [False, True])
def test_teacher_forced_scoring(model_folders, dtype, decode_step):
    """Negative log-likelihood of given tokens, through the prompt step (in pieces) or token by token,
    against the plain logits' log-softmax; three sequences of unequal lengths as one batch."""
    import supersonic_b200
    from supersonic_b200.engine.score import teacher_forced
    d, pc, pw = model_folders["C"]
    rng = np.random.default_rng(61)
    seqs = [rng.integers(0, pc["vocab_size"], n).tolist() for n in (40, 2, 17)]
    eng = supersonic_b200.load(d, dtype=dtype, context_size=64, batch_size=3)
    got = teacher_forced(eng.model, seqs, decode_step=decode_step, rows_per_step=16)
    for s, g in zip(seqs, got):
        logits = pl.forward(pc, pw, s)[:-1]
        m = logits.max(axis=1, keepdims=True)
        nll = (m[:, 0] + np.log(np.exp(logits - m).sum(axis=1))) - logits[np.arange(len(s) - 1), s[1:]]
        assert g.scored_tokens == len(s) - 1 and g.tokens == len(s)
        tol = 2e-5 if dtype == "float32" else 2e-2 * np.abs(logits).max()
        assert abs(g.avg_nll - nll.mean()) < tol
        assert abs(g.perplexity - np.exp(nll.mean())) < 2 * tol * np.exp(nll.mean())
        assert g.decode_steps == (len(s) - 2 if decode_step else 0)
    assert eng.model.cache.slots.n_held == 0
    assert eng.score(seqs[:1])[0].scored_tokens == 39


def test_command_line_teacher_forced(model_folders):
    import json
    d, pc, pw = model_folders["A"]
    seq = np.random.default_rng(62).integers(0, 256, 20).tolist()
    proc = _run_cli("--model-dir", d, "--prompt-ids", ",".join(map(str, seq)), "--teacher-forced", "--dtype", "float32")
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("[teacher_forced_json] ")][0]
    rec = json.loads(line[len("[teacher_forced_json] "):])
    logits = pl.forward(pc, pw, seq)[:-1]
    m = logits.max(axis=1, keepdims=True)
    nll = (m[:, 0] + np.log(np.exp(logits - m).sum(axis=1))) - logits[np.arange(19), seq[1:]]
    assert rec["scored_tokens"] == 19 and abs(rec["total_nll"] - nll.sum()) < 1e-3
    assert abs(rec["perplexity"] - np.exp(nll.mean())) < 1e-3 and "[teacher_forced] tokens=20" in proc.stderr


def test_a_folder_with_buffer_tensors_loads(tmp_path):
    """``rotary_emb.inv_freq`` buffers that some exporters store are passed over; any other tensor the
    configuration does not name is an error that lists it, or a warning if the caller says so."""
    import tiny_configs
    import warnings
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.engine import Model
    from supersonic_b200.weights import WeightError, random_tensors, write_safetensors
    cfg = config_from_dict(tiny_configs.A)
    tensors = dict(random_tensors(cfg, 0))
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    import json
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(tmp_path / "model.safetensors"), [(n, t.dtype, list(t.shape)) for n, t in tensors.items()],
                      iter(tensors.items()))
    Model.from_dir(str(tmp_path), dtype="float32", max_tokens=64)
    tensors["model.extra.weight"] = torch.ones(3)
    write_safetensors(str(tmp_path / "model.safetensors"), [(n, t.dtype, list(t.shape)) for n, t in tensors.items()],
                      iter(tensors.items()))
    with pytest.raises(WeightError, match="unexpected .*model.extra.weight"):
        Model.from_dir(str(tmp_path), dtype="float32", max_tokens=64)
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        Model.from_dir(str(tmp_path), dtype="float32", max_tokens=64, allow_unexpected_tensors=True)
    assert any("model.extra.weight" in str(w.message) for w in seen)


@pytest.mark.parametrize("name", ["D", "E"])
def test_bfloat16_sampling_is_reproducible_in_deterministic_mode(model_folders, name):
    """bfloat16 with ``deterministic=True`` (no float atomics; a sequence's keys are cut the same way
    in every batch): the same seed gives the same tokens twice, in a batch of four, in pairs and
    alone; and the logits of a sequence are the same bits alone and among others."""
    import supersonic_b200
    from supersonic_b200.engine import StepEntry
    d, pc, pw = model_folders[name]
    rng = np.random.default_rng(71)
    prompts = [rng.integers(0, pc["vocab_size"], n).tolist() for n in (9, 3, 150, 70)]
    eng = supersonic_b200.load(d, dtype="bfloat16", context_size=256, batch_size=4, deterministic=True)
    assert eng.model.kernels.deterministic and eng.model.use_graphs
    kw = dict(max_new_tokens=24, temperature=0.8, top_k=50, sampling_seed=1234, ignore_eos=True)
    together = eng.generate(prompts, batch_size=4, **kw)
    assert together == eng.generate(prompts, batch_size=4, **kw)          # the seed decides, every time
    assert eng.generate(prompts, batch_size=2, **kw) == together          # the batch does not
    assert [eng.generate([p], batch_size=1, **{**kw, "sampling_seed": 1234})[0] for p in prompts[:1]] == together[:1]
    assert eng.generate(prompts, batch_size=4, **{**kw, "sampling_seed": 99}) != together
    # logits, bit for bit: a sequence alone against the same sequence among three others, prompt and decode
    m = eng.model
    slots = [m.open_sequence() for _ in prompts]
    batch = m.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    nxt = [int(t) for t in batch.argmax(-1)]
    batch2 = m.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt)])
    for s in slots:
        m.close_sequence(s)
    for i in (0, 2):
        s = m.open_sequence()
        alone = m.step([StepEntry(s, prompts[i], [len(prompts[i]) - 1])])
        alone2 = m.step([StepEntry(s, [nxt[i]], [0])])
        m.close_sequence(s)
        assert torch.equal(alone[0], batch[i]), f"prompt {i}"
        assert torch.equal(alone2[0], batch2[i]), f"decode {i}"


@pytest.mark.parametrize("name", ["B", "E"])
def test_prompt_steps_of_recurring_sizes_are_captured_and_stay_right(model_folders, name):
    """The second time a prompt step of the same sizes comes up it is recorded as a graph, the third
    time replayed: other tokens, other slots, other pages each time, the logits those of the plain
    implementation.  A step in pieces (a small token budget) recurs by construction."""
    from supersonic_b200.engine import Model, StepEntry
    d, pc, pw = model_folders[name]
    rng = np.random.default_rng(91)
    m = Model.from_dir(d, dtype="bfloat16", max_tokens=2048)
    assert m.use_prompt_graphs
    held = []
    for round_ in range(4):
        a = rng.integers(0, pc["vocab_size"], 130).tolist()
        b = rng.integers(0, pc["vocab_size"], 37).tolist()
        if round_ == 2:
            held.append(m.open_sequence())               # shifts the slots and pages the next rounds get
        sa, sb = m.open_sequence(), m.open_sequence()
        got = m.step([StepEntry(sa, a, [0, 129]), StepEntry(sb, b, [36])]).double().cpu().numpy()
        ra, rb = pl.forward(pc, pw, a), pl.forward(pc, pw, b)
        want = np.stack([ra[0], ra[129], rb[36]])
        assert np.abs(got - want).max() < 2e-2 * np.abs(want).max(), round_
        nxt = m.step([StepEntry(sa, [5], [0]), StepEntry(sb, [6], [0])]).double().cpu().numpy()     # the cache it left is right
        wa, wb = pl.forward(pc, pw, a + [5])[-1], pl.forward(pc, pw, b + [6])[-1]
        assert np.abs(nxt - np.stack([wa, wb])).max() < 2e-2 * max(np.abs(wa).max(), np.abs(wb).max())
        m.close_sequence(sa); m.close_sequence(sb)
    assert m.prompt_graph_replays == 3 and len(m._prompt_graphs) == 1
    m.check_errors()
    # in pieces: 300 tokens with a budget of 64 are four steps of 64 tokens and one of 44; by the second
    # prompt every size has come up before
    m2 = Model.from_dir(d, dtype="bfloat16", max_tokens=1024, step_token_budget=64)
    for round_ in range(2):
        t = rng.integers(0, pc["vocab_size"], 300).tolist()
        s = m2.open_sequence()
        got = m2.step([StepEntry(s, t, [299])]).double().cpu().numpy()
        want = pl.forward(pc, pw, t)[-1]
        assert np.abs(got[0] - want).max() < 2e-2 * np.abs(want).max()
        m2.close_sequence(s)
    assert m2.prompt_graph_replays >= 4
