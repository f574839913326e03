"""The workload of a whole small model at real widths: Llama-3.2-1B sizes with random bfloat16
weights, a ragged batch of 64 prompts of 1 to 4,096 tokens through the Python entry point with
temperature sampling, then a float32 replay of four of the sequences beside the bfloat16 one.

No plain reference runs at this size (it would take minutes on the CPU); what is checked is what
can only go wrong at size: every sequence gets its tokens, the cache gives every slot and page
back, and the bfloat16 logits stay within rounding noise of
the float32 path's at every replayed position (a wrong page, a wrong split or a stale slot shows as
a row that is off by the size of the logits themselves).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N_SEQS, MAX_PROMPT, NEW = 64, 4096, 48


def _build(cfg, dtype, max_tokens, ctx):
    from supersonic_b200.engine import Model
    from supersonic_b200.weights import RandomWeightStore
    store = RandomWeightStore(cfg, seed=4, device="cuda:0", std=0.02, norm_jitter=0.0)
    return Model.from_config(cfg, store, dtype=dtype, device="cuda:0", max_tokens=max_tokens, max_seq_tokens=ctx)


def test_ragged_batch_of_64_at_1b_sizes_and_float32_replay():
    from supersonic_b200.api import Engine
    from supersonic_b200.config import preset_config
    from supersonic_b200.engine import StepEntry
    cfg = preset_config("llama3.2-1b")
    rng = np.random.default_rng(4)
    lens = rng.integers(1, MAX_PROMPT + 1, N_SEQS).tolist()
    lens[0], lens[1] = 1, MAX_PROMPT                                   # both ends of the range are present
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in lens]
    ctx = -(-(MAX_PROMPT + NEW) // 64) * 64
    model = _build(cfg, "bfloat16", N_SEQS * ctx, ctx)
    eng = Engine(model)
    kw = dict(max_new_tokens=NEW, temperature=1.0, sampling_seed=7, ignore_eos=True, batch_size=N_SEQS)
    out = eng.generate(prompts, **kw)
    assert [len(o) for o in out] == [NEW] * N_SEQS
    assert all(0 <= t < cfg.vocab_size for o in out for t in o)
    assert model.cache.slots.n_held == 0
    model.cache.check()
    # once more over the slots and pages that were given back (the tokens are not compared: the
    # residual adds with float atomics, so two bfloat16 runs differ by rounding and a sample may flip)
    again = eng.generate(prompts[::-1], **kw)
    assert [len(o) for o in again] == [NEW] * N_SEQS and model.cache.slots.n_held == 0
    model.cache.check()
    assert len({tuple(o) for o in out}) == N_SEQS                      # sequences are not copies of one another
    del eng, model
    torch.cuda.empty_cache()

    order = sorted(range(N_SEQS), key=lambda i: lens[i])
    pick = [order[0], order[N_SEQS // 3], order[2 * N_SEQS // 3], order[-1]]
    logits = {}
    for dtype in ("bfloat16", "float32"):
        m = _build(cfg, dtype, 4 * ctx, ctx)
        slots = [m.open_sequence() for _ in pick]
        rows = [m.step([StepEntry(s, prompts[i], [lens[i] - 1]) for s, i in zip(slots, pick)]).float().cpu()]
        for t in range(12):
            rows.append(m.step([StepEntry(s, [out[i][t]], [0]) for s, i in zip(slots, pick)]).float().cpu())
        logits[dtype] = torch.stack(rows).double()                     # [13 steps, 4 sequences, vocab]
        for s in slots:
            m.close_sequence(s)
        m.cache.check()
        del m
        torch.cuda.empty_cache()
    ref, got = logits["float32"], logits["bfloat16"]
    assert torch.isfinite(ref).all() and torch.isfinite(got).all()
    # per position: the error's root mean square against the spread of the logits themselves.
    # bfloat16 activations through 16 layers leave about 2 %; a fault leaves about 100 %.
    rel = (got - ref).pow(2).mean(-1).sqrt() / ref.std(-1)
    assert float(rel.max()) < 0.05, rel
    assert float((got - ref).abs().max()) < 0.05 * float(ref.abs().max())
