"""The generation loop's decisions, on the CPU with a scripted model: batches of unequal
prompts, stop tokens, sequences that end early, one batch after another in reused slots."""
import pytest
import torch

from supersonic_b200.cache import KvNeed, SequenceCache
from supersonic_b200.engine.generate import Generator, finished, plan_batch
from supersonic_b200.sampling import SamplingParams, request_seed


class ScriptedModel:
    """Next token = (sum of the sequence's tokens) % vocab: depends on the whole history of
    the right sequence, so any mix-up of slots or tokens shows."""

    class _Spec:
        stop_token_ids = [3]

    def __init__(self, vocab=11, max_tokens=64 * 4, max_seq=128, max_slots=None):
        self.vocab, self.spec, self.device = vocab, self._Spec(), "cpu"
        self.kernels = None
        self.cache = SequenceCache({0: KvNeed(1, 16)}, max_tokens, max_seq, torch.float32, "cpu", max_slots)
        self.history = {}
        self.step_sizes = []
        self.slots_seen = []

    def open_sequence(self, seed=None):
        s = self.cache.acquire(seed)
        self.history[s] = []
        self.slots_seen.append(s)
        return s

    def close_sequence(self, s):
        self.cache.release(s)
        del self.history[s]

    def step(self, entries):
        self.step_sizes.append([len(e.tokens) for e in entries])
        rows = []
        for e in entries:
            self.cache.reserve(e.slot, len(e.tokens)); self.cache.advance(e.slot, len(e.tokens))
            self.history[e.slot].extend(e.tokens)
            assert len(self.history[e.slot]) == self.cache.length(e.slot)
            for w in e.want:
                assert w == len(e.tokens) - 1
                row = torch.zeros(self.vocab)
                row[sum(self.history[e.slot]) % self.vocab] = 1.0
                rows.append(row)
        return torch.stack(rows)


class ScriptedModelAhead(ScriptedModel):
    """The same model with the interface of a device that runs one step ahead of the host: tokens of a
    step may come as a tensor (here on the CPU), and reading them back is split in two."""

    feeds_device_tokens = True

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.device = torch.device("cpu")
        self.ahead_steps = 0

    def step_ahead(self, slots, tokens):
        from supersonic_b200.engine import StepEntry
        assert isinstance(tokens, torch.Tensor) and tokens.dtype == torch.int32 and tokens.numel() == len(slots)
        self.ahead_steps += 1
        return self.step([StepEntry(s, [int(t)], [0]) for s, t in zip(slots, tokens.tolist())])

    def start_fetch(self, values):
        return values.clone()

    def finish_fetch(self, handle):
        return handle.tolist()


MODELS = [ScriptedModel, ScriptedModelAhead]


def greedy(logits, slots, params):
    return logits.argmax(-1).to(torch.int32)


def expected(prompt, n, vocab=11, stop=(3,), include_stop=True):
    toks, out = list(prompt), []
    while len(out) < n:
        t = sum(toks) % vocab
        toks.append(t)
        if t in stop:
            if include_stop:
                out.append(t)
            return out, "stop"
        out.append(t)
    return out, "length"


def test_finished_rules():
    assert finished(3, 1, 8, {3}) == "stop"
    assert finished(4, 8, 8, {3}) == "length"
    assert finished(4, 7, 8, {3}) is None
    assert finished(3, 8, 8, {3}) == "stop"          # a stop token at the budget is still a stop


def test_plan_batch_respects_pages_slots_and_batch_size():
    lens = [10, 100, 30, 64]
    assert plan_batch([0, 1, 2, 3], lens, 8, 64 * 4, 8, 64, None) == [0, 1, 2]     # 64+128+64 fit, 128 more not
    assert plan_batch([0, 1, 2, 3], lens, 8, 64 * 100, 2, 64, None) == [0, 1]      # slots
    assert plan_batch([0, 1, 2, 3], lens, 8, 64 * 100, 8, 64, 3) == [0, 1, 2]      # batch size
    assert plan_batch([1], lens, 8, 64, 8, 64, None) == []                         # does not fit at all


@pytest.mark.parametrize("Model", MODELS)
def test_unequal_prompts_early_ends_and_slot_reuse(Model):
    m = Model(max_tokens=64 * 3, max_seq=128)
    g = Generator(m, sampler=greedy)
    prompts = [[1, 2], [5, 6, 7, 8, 9], [2], [4, 4, 4], [10, 1, 1, 1, 1, 1, 1], [6]]
    res = g.generate(prompts, max_new_tokens=6, batch_size=3)
    for p, r in zip(prompts, res):
        want, why = expected(p, 6)
        assert r.tokens == want and r.finish_reason == why and r.prompt_tokens == len(p)
    # first step of each batch brings whole prompts, later steps one token per live sequence
    assert m.step_sizes[0] == [2, 5, 1]
    assert all(all(n == 1 for n in s) for s in m.step_sizes[1:] if s != [3, 7, 1])
    assert [3, 7, 1] in m.step_sizes                       # second batch started together
    assert sorted(set(m.slots_seen)) == [0, 1, 2] and len(m.slots_seen) == 6      # slots used again
    assert m.cache.slots.n_held == 0 and m.cache.free_tokens() == 64 * 3
    m.cache.check()
    # steps shrink as sequences end
    sizes = [len(s) for s in m.step_sizes]
    assert any(a > b for a, b in zip(sizes, sizes[1:]))
    if Model is ScriptedModelAhead:
        assert m.ahead_steps > 0                           # the loop did run ahead
        # a sequence that ends at a stop token was stepped once more than the simple loop steps it;
        # one that ends at its budget was not
        simple = ScriptedModel(max_tokens=64 * 3, max_seq=128)
        Generator(simple, sampler=greedy).generate(prompts, max_new_tokens=6, batch_size=3)
        stops = sum(1 for p in prompts if expected(p, 6)[1] == "stop" and len(expected(p, 6)[0]) < 6)
        assert sum(sizes) - sum(len(x) for x in simple.step_sizes) == stops


@pytest.mark.parametrize("Model", MODELS)
def test_stop_token_options_and_zero_budget(Model):
    prompts = [[1, 2], [7, 7]]
    m = Model()
    g = Generator(m, sampler=greedy)
    res = g.generate(prompts, max_new_tokens=5, include_stop_token=False)
    assert [r.tokens for r in res] == [expected(p, 5, include_stop=False)[0] for p in prompts]
    res = g.generate(prompts, max_new_tokens=5, ignore_eos=True)
    assert all(len(r.tokens) == 5 and r.finish_reason == "length" for r in res)
    res = g.generate(prompts, max_new_tokens=5, stop_token_ids=[9])
    assert [r.tokens for r in res] == [expected(p, 5, stop=(9,))[0] for p in prompts]
    before = len(m.step_sizes)
    res = g.generate(prompts, max_new_tokens=0)
    assert [r.tokens for r in res] == [[], []] and len(m.step_sizes) == before + 1   # the prompt still runs
    assert m.cache.slots.n_held == 0


@pytest.mark.parametrize("Model", MODELS)
def test_requests_that_cannot_fit_are_refused(Model):
    m = Model(max_tokens=64 * 2, max_seq=128)
    g = Generator(m, sampler=greedy)
    with pytest.raises(ValueError, match="exceed"):
        g.generate([[1] * 125], max_new_tokens=8)
    with pytest.raises(ValueError, match="empty"):
        g.generate([[]])
    assert m.cache.slots.n_held == 0


@pytest.mark.parametrize("Model", MODELS)
def test_a_failing_step_gives_slots_back(Model):
    m = Model()
    calls = []

    def bad_sampler(logits, slots, params):
        calls.append(1)
        if len(calls) == 2:
            raise RuntimeError("boom")
        return greedy(logits, slots, params)
    with pytest.raises(RuntimeError, match="boom"):
        Generator(m, sampler=bad_sampler).generate([[1, 2], [2, 2]], max_new_tokens=5, ignore_eos=True)
    assert m.cache.slots.n_held == 0
    m.cache.check()


def test_request_seeds_differ_and_are_stable():
    seeds = {request_seed(42, i) for i in range(100)}
    assert len(seeds) == 100 and 0 not in seeds and request_seed(42, 3) == request_seed(42, 3)
    assert request_seed(42, 0) != request_seed(43, 0)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    assert SamplingParams().greedy and SamplingParams(temperature=0.7, top_k=1).greedy
    assert not SamplingParams(temperature=0.7).greedy


def test_a_long_step_is_cut_into_chunks_that_keep_order_and_budget():
    """The planner of a step that exceeds its token budget: every token once, in order, no chunk
    over the budget, no entry twice in a chunk, no empty chunk."""
    import random
    from supersonic_b200.engine.batch import plan_chunks
    assert plan_chunks([5, 3], 100) == [[(0, 0, 5), (1, 0, 3)]]
    assert plan_chunks([5, 3], 4) == [[(0, 0, 4)], [(0, 4, 5), (1, 0, 3)]]
    assert plan_chunks([4, 4], 4) == [[(0, 0, 4)], [(1, 0, 4)]]
    assert plan_chunks([1, 9, 1], 3) == [[(0, 0, 1), (1, 0, 2)], [(1, 2, 5)], [(1, 5, 8)], [(1, 8, 9), (2, 0, 1)]]
    with pytest.raises(ValueError):
        plan_chunks([3], 0)
    rnd = random.Random(5)
    for _ in range(200):
        counts = [rnd.randint(1, 40) for _ in range(rnd.randint(1, 9))]
        budget = rnd.randint(1, 50)
        chunks = plan_chunks(counts, budget)
        seen = [[] for _ in counts]
        for c in chunks:
            assert c and sum(hi - lo for _, lo, hi in c) <= budget
            assert len({i for i, _, _ in c}) == len(c)
            assert [i for i, _, _ in c] == sorted(i for i, _, _ in c)
            for i, lo, hi in c:
                assert lo < hi
                seen[i].append((lo, hi))
        for n, parts in zip(counts, seen):
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        # full chunks except the last
        assert all(sum(hi - lo for _, lo, hi in c) == budget for c in chunks[:-1])


def test_which_gemm_a_prompt_gets_is_decided_by_its_rows():
    """The dispatch rules of the prefill projections are plain functions of the sizes: tiles on SM
    pairs where the second half of the last 256 rows is not mostly padding, K cut into parts only
    while the tiles alone leave SMs idle."""
    from supersonic_b200.csrc.fast_sets import FastKernels as FK
    assert FK._pair_tiles(2048, 6144) and FK._pair_tiles(512, 28672) and FK._pair_tiles(1030, 4096)
    assert FK._pair_tiles(256, 256) and FK._pair_tiles(200, 4096)        # two row tiles of 128
    assert not FK._pair_tiles(300, 28672) and not FK._pair_tiles(100, 4096) and not FK._pair_tiles(2048, 128)
    assert FK._gemm_splits(2048, 4096, 4096, 256, 148) == 1                    # 256 tiles: more than the SMs
    assert FK._gemm_splits(128, 4096, 14336, 256, 148) == 9                    # 16 tiles, 224 k-blocks
    assert FK._gemm_splits(128, 4096, 4096, 256, 148) == 8                     # at least 8 k-blocks a part
    assert FK._gemm_splits(70, 256, 192, 256, 148) == 1                        # a tiny model: K is too short to cut
    assert FK._tile_n(2048, 4096) == 256 and FK._tile_n(8, 4096) == 64 and FK._tile_n(8, 128256) == 256


def test_command_line_helpers(tmp_path):
    from supersonic_b200 import cli
    assert cli.parse_ids("1, 2,3 4") == [1, 2, 3, 4]
    f = tmp_path / "p.txt"
    f.write_text("# header\n1,2,3\n\n 7 8 9 # tail\n")
    assert cli.read_prompt_file(str(f)) == [[1, 2, 3], [7, 8, 9]]
    f.write_text("1,two\n")
    with pytest.raises(ValueError, match="p.txt:1"):
        cli.read_prompt_file(str(f))
    ap = cli.build_parser()
    a = ap.parse_args(["--preset", "tiny-a", "--random-seed", "3", "--stop-ids", "5,6", "--prompt-file", "x"])
    assert a.preset == "tiny-a" and a.random_seed == 3 and a.stop_ids == "5,6" and a.prompt_file == ["x"]
    # refusals that need no device
    assert cli.main(["--prompt-ids", "1,2"]) == 2
    assert cli.main(["--preset", "nope", "--prompt-ids", "1"]) == 2
    assert cli.main(["--preset", "tiny-a", "--prompt-ids", "1,2,3", "--context-size", "4"]) == 2
    assert cli.main(["--preset", "tiny-a"]) == 2
