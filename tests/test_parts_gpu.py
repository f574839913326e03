"""Each part alone against the plain implementation, the order of layers as data (a layer
twice, a layer reading another layer's cache, a window), and a toy mixer with state of its
own that is registered, built and stepped without touching the framework."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build_ctx(dtype, store=None, max_positions=512):
    from supersonic_b200.csrc.kernel_sets import kernel_set_for
    from supersonic_b200.parts import BuildContext, WeightAccess
    from supersonic_b200.weights import WeightStore
    store = store or WeightStore.from_tensors({})
    return BuildContext(torch.device(DEV), dtype, kernel_set_for(dtype), WeightAccess(store, DEV), max_positions)


def step_ctx(build, cache, entries):
    from supersonic_b200.engine import StepContext, pack_step
    starts = [cache.length(e.slot) for e in entries]
    batch = pack_step(entries, starts, DEV)
    for e in entries:
        cache.reserve(e.slot, len(e.tokens))
    cache.sync()
    return StepContext(batch, cache, build.kernels, build.dtype)


def tolerance(dtype, scale=1.0):
    return 2e-5 * max(scale, 1.0) if dtype == torch.float32 else 2e-2 * max(scale, 1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_embedding_head(dtype):
    from supersonic_b200.parts import EMBEDDINGS, HEADS, NORMS
    from supersonic_b200.weights import WeightStore
    g = torch.Generator().manual_seed(0)
    w = {"n": (1 + 0.1 * torch.randn(72, generator=g)).bfloat16(), "e": torch.randn(301, 72, generator=g).bfloat16()}
    b = build_ctx(dtype, WeightStore.from_tensors(w))
    norm = NORMS["rmsnorm"]({"size": 72, "eps": 2e-5}, {"weight": "n"}, b)
    emb = EMBEDDINGS["embedding"]({"vocab_size": 301, "hidden_size": 72}, {"weight": "e"}, b)
    head = HEADS["linear_head"]({"vocab_size": 301, "hidden_size": 72}, {"weight": "e"}, b)
    assert head.weight.data_ptr() == emb.table.data_ptr()               # tied: one buffer
    ctx = type("C", (), {"kernels": b.kernels})()
    ids = torch.tensor([3, 300, 0, 3], dtype=torch.int32, device=DEV)
    h = emb(ctx, ids)
    wn, we = w["n"].double().numpy(), w["e"].double().numpy()
    assert h.dtype == torch.float32 and np.allclose(h.cpu().numpy(), pl.embedding(ids.tolist(), we))
    n = norm(ctx, h)
    ref = pl.rms_norm(pl.embedding(ids.tolist(), we), wn, 2e-5)
    assert n.dtype == dtype and np.abs(n.double().cpu().numpy() - ref).max() < tolerance(dtype, np.abs(ref).max())
    rows = torch.tensor([2, 1], dtype=torch.int32, device=DEV)
    logits = head(ctx, norm(ctx, h, rows=rows))
    ref_l = ref[[2, 1]] @ we.T
    assert logits.dtype == torch.float32 and tuple(logits.shape) == (2, 301)
    assert np.abs(logits.double().cpu().numpy() - ref_l).max() < tolerance(dtype, np.abs(ref_l).max())


def test_rotary_tables_match_plain():
    from supersonic_b200.parts import POSITION_ENCODINGS
    for cfg in (tiny_configs.A, tiny_configs.B, tiny_configs.C):
        hd = cfg["head_dim"]
        rot = POSITION_ENCODINGS["rotary"](
            {"head_dim": hd, "rotary_dim": hd, "theta": cfg["rope_theta"], "max_positions": 400,
             "scaling": cfg["rope_scaling"]}, {}, build_ctx(torch.float32))
        cos, sin = pl.rope_tables(cfg, 400)
        assert np.abs(rot.cos.double().cpu().numpy() - cos).max() < 1e-7
        assert np.abs(rot.sin.double().cpu().numpy() - sin).max() < 1e-7


def _layer_weights(cfg, seed, std=0.1):
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import random_store
    c = config_from_dict(cfg)
    return c, random_store(c, seed, std=std)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "C"])
def test_mixer_feed_forward_and_block_alone(dtype, name):
    """Layer 0's parts built by hand and run over a prompt, then token by token."""
    from supersonic_b200.cache import SequenceCache
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
    cfg, seed, std = tiny_configs.CONFIGS[name]
    c, store = _layer_weights(cfg, seed, std)
    pw = {n: store.get(n).double().numpy() for n in store.names()}
    spec = c.build_spec().blocks[0]
    b = build_ctx(dtype, store)
    mixer = MIXERS[spec.mixer.kind](spec.mixer.params, spec.mixer.weights, b)
    ff = FEED_FORWARDS[spec.feed_forward.kind](spec.feed_forward.params, spec.feed_forward.weights, b)
    n1 = NORMS["rmsnorm"](spec.mixer_norm.params, spec.mixer_norm.weights, b)
    n2 = NORMS["rmsnorm"](spec.feed_forward_norm.params, spec.feed_forward_norm.weights, b)
    pos = POSITION_ENCODINGS[spec.position.kind](spec.position.params, spec.position.weights, b)
    cache = SequenceCache({0: mixer.cache_need()}, 512, 256, dtype, DEV)
    T, H = 75, c.hidden_size
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(3))
    xd = x.double().numpy()
    cos, sin = pl.rope_tables(cfg, T)
    ref_mix = pl.attention_mixer(xd, pw, "model.layers.0", cfg, cos, sin)
    ref_ff = pl.swiglu_ffn(xd, pw, "model.layers.0")
    ref_block = pl.block(xd, pw, 0, cfg, cos, sin)

    # feed-forward alone
    ctx = type("C", (), {"kernels": b.kernels})()
    res = torch.zeros(T, H, device=DEV)
    ff.forward(ctx, x.to(DEV, dtype), res)
    xq = x.to(dtype).double().numpy()                 # the part sees activations already rounded
    ref_ffq = pl.swiglu_ffn(xq, pw, "model.layers.0")
    assert np.abs(res.double().cpu().numpy() - ref_ffq).max() < tolerance(dtype, np.abs(ref_ff).max())

    # mixer alone: 70 tokens at once, then 5 one by one, against whole-sequence plain attention
    slot = cache.acquire()
    ref_mixq = pl.attention_mixer(xq, pw, "model.layers.0", cfg, cos, sin)
    got = []
    for lo, hi in [(0, 70)] + [(i, i + 1) for i in range(70, 75)]:
        sc = step_ctx(b, cache, [StepEntry(slot, [0] * (hi - lo))])
        res = torch.zeros(hi - lo, H, device=DEV)
        mixer.forward(sc, x[lo:hi].to(DEV, dtype), res, 0, True, pos)
        cache.advance(slot, hi - lo)
        got.append(res)
    got = torch.cat(got).double().cpu().numpy()
    assert np.abs(got - ref_mixq).max() < tolerance(dtype, np.abs(ref_mix).max())
    cache.release(slot)

    # the block arrangement
    block = BLOCKS[spec.kind](mixer, ff, n1, n2, pos)
    slot = cache.acquire()
    res = x.to(DEV).clone()
    sc = step_ctx(b, cache, [StepEntry(slot, [0] * T)])
    block.forward(sc, res, 0, True)
    assert np.abs(res.double().cpu().numpy() - ref_block).max() < tolerance(dtype, np.abs(ref_block).max())


def _spec_with(cfg, schedule=None, window=None):
    from dataclasses import replace
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.config.base import PartSpec
    spec = config_from_dict(cfg).build_spec()
    blocks = list(spec.blocks)
    if window is not None:
        for i, w in window.items():
            m = blocks[i].mixer
            blocks[i] = replace(blocks[i], mixer=PartSpec(m.kind, {**m.params, "window": w}, m.weights))
    return replace(spec, blocks=blocks, schedule=schedule or spec.schedule)


def _plain_forward_scheduled(cfg, pw, tokens, schedule, window=None):
    """The plain parts run in the order a schedule gives; a stop that does not write a cache
    attends with its own queries over the keys and values of the stop that wrote it."""
    T = len(tokens)
    cos, sin = pl.rope_tables(cfg, T)
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    h = pl.embedding(tokens, pw["model.embed_tokens.weight"])
    kv = {}
    for layer, cache, writes in schedule:
        p = f"model.layers.{layer}"
        x = pl.rms_norm(h, pw[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        q = pl.apply_rope((x @ pw[f"{p}.self_attn.q_proj.weight"].T).reshape(T, nq, hd), cos, sin)
        if writes:
            k = pl.apply_rope((x @ pw[f"{p}.self_attn.k_proj.weight"].T).reshape(T, nkv, hd), cos, sin)
            kv[cache] = (k, (x @ pw[f"{p}.self_attn.v_proj.weight"].T).reshape(T, nkv, hd))
        k, v = kv[cache]
        a = pl.attention_scores(q, k, v, 1 / math.sqrt(hd), (window or {}).get(layer)).reshape(T, nq * hd)
        h = h + a @ pw[f"{p}.self_attn.o_proj.weight"].T
        h = h + pl.swiglu_ffn(pl.rms_norm(h, pw[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"]), pw, p)
    return pl.output_head(h, pw, cfg)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_order_of_layers_is_data(dtype, model_folders):
    """Layer 1 twice (each time with a cache entry of its own), layer 0 reading the cache that
    layer 2 wrote, and a window on layer 1: whole prompt, then token by token."""
    from supersonic_b200.config.base import ScheduleEntry
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import WeightStore
    d, pc, pw = model_folders["B"]
    order = [(0, 0, True), (1, 1, True), (2, 2, True), (2, 2, False), (1, 3, True)]
    window = {1: 9}
    # layer 2 reads its own cache a second time without writing: the same need by construction
    spec = _spec_with(tiny_configs.B, [ScheduleEntry(l, c, w) for l, c, w in order], window)
    m = Model(spec, WeightStore.from_dir(d), dtype=dtype, device=DEV, max_tokens=256)
    assert len(m.cache.kv_groups) == 2                                   # full and windowed storage
    toks = np.random.default_rng(5).integers(0, 384, 90).tolist()
    ref = _plain_forward_scheduled(pc, pw, toks, order, window)
    s = m.open_sequence()
    got = [m.step([StepEntry(s, toks[:80], range(80))])]
    got += [m.step([StepEntry(s, [toks[p]], [0])]) for p in range(80, 90)]
    got = torch.cat(got).double().cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 2e-2 * np.abs(ref).max()
    assert np.abs(got - ref).max() < tol
    m.cache.check()
    win = next(g for g in m.cache.kv_groups if g.need.window)
    assert len(win.held[s]) == 1 and min(win.held[s]) == 1              # the window group dropped page 0


def _tol(dtype, ref):
    return 2e-5 if dtype == "float32" else 2e-2 * np.abs(ref).max()


@pytest.mark.parametrize("dtype,on_device", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_toy_mixer_with_its_own_state(dtype, on_device, model_folders):
    """A mixer defined here, with a fixed-size state per sequence instead of keys and values,
    is registered, built into a model and stepped: nothing in the framework's files changes.
    In bfloat16 it runs beside the serving kernels.  One variant reads the batch's host lists and
    says so (``capture_safe = False``: the model then steps uncaptured); the other takes a decode
    step from the batch's device tensors alone and is replayed inside the captured graphs."""
    from dataclasses import replace
    from supersonic_b200.cache import StateNeed
    from supersonic_b200.config.base import PartSpec
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.parts import register_mixer
    from supersonic_b200.weights import WeightStore

    @register_mixer("toy_decay")
    class ToyDecay:
        """s <- decay * s + x_t ; out_t = s W^T.  State: one float32 vector per sequence."""

        capture_safe = "decode" if on_device else False     # its prompt steps read the batch's host lists

        def __init__(self, params, weights, build):
            self.hidden, self.decay = params["hidden_size"], params["decay"]
            self.w = build.weights.as_dtype(weights["w"], torch.float32)

        def cache_need(self):
            return StateNeed(self.hidden)

        def forward(self, ctx, x, residual, cache_id, writes_cache, position):
            state = ctx.cache.state(cache_id)
            b, row = ctx.batch, 0
            if on_device and b.is_decode:
                # one token a sequence, everything from device tensors; rows whose slot is negative
                # (a captured step's warm-up) change nothing
                live = (b.seq_slot >= 0)[:, None]
                idx = b.seq_slot.clamp(min=0).long()
                old = state[idx]
                new = torch.where(live, self.decay * old + x.float(), old)
                state.index_copy_(0, idx, new)
                residual += torch.where(live, new @ self.w.T, torch.zeros_like(residual))
                return
            for slot, n in zip(b.host_slots, b.host_counts):
                s = state[slot]
                for t in range(row, row + n):
                    s = self.decay * s + x[t].float()
                    residual[t] += s @ self.w.T
                state[slot] = s
                row += n

    d, pc, pw = model_folders["A"]
    spec = _spec_with(tiny_configs.A)
    toy = PartSpec("toy_decay", {"hidden_size": 64, "decay": 0.5}, {"w": "model.layers.1.self_attn.o_proj.weight"})
    spec = replace(spec, blocks=[spec.blocks[0], replace(spec.blocks[1], mixer=toy, position=None)])
    m = Model(spec, WeightStore.from_dir(d), dtype=dtype, device=DEV, max_tokens=256)
    assert len(m.cache.kv_groups) == 1 and tuple(m.cache.state(1).shape)[1] == 64
    assert m.use_graphs == (dtype == "bfloat16" and on_device)

    def plain(tokens):
        T = len(tokens)
        cos, sin = pl.rope_tables(pc, T)
        h = pl.block(pl.embedding(tokens, pw["model.embed_tokens.weight"]), pw, 0, pc, cos, sin)
        x = pl.rms_norm(h, pw["model.layers.1.input_layernorm.weight"], pc["rms_norm_eps"])
        s, outs = np.zeros(64), []
        for t in range(T):
            s = 0.5 * s + x[t]
            outs.append(s @ pw["model.layers.1.self_attn.o_proj.weight"].T)
        h = h + np.stack(outs)
        h = h + pl.swiglu_ffn(pl.rms_norm(h, pw["model.layers.1.post_attention_layernorm.weight"],
                                          pc["rms_norm_eps"]), pw, "model.layers.1")
        return pl.output_head(h, pw, pc)

    rng = np.random.default_rng(6)
    a, b = rng.integers(0, 256, 20).tolist(), rng.integers(0, 256, 9).tolist()
    sa, sb = m.open_sequence(), m.open_sequence()
    got = m.step([StepEntry(sa, a[:15], range(15)), StepEntry(sb, b[:4], range(4))])
    ga, gb = [got[:15]], [got[15:]]
    for i in range(5):
        got = m.step([StepEntry(sa, [a[15 + i]], [0]), StepEntry(sb, [b[4 + i]], [0])])
        ga.append(got[:1]); gb.append(got[1:])
    assert np.abs(torch.cat(ga).double().cpu().numpy() - plain(a)).max() < _tol(dtype, plain(a))
    assert np.abs(torch.cat(gb).double().cpu().numpy() - plain(b)).max() < _tol(dtype, plain(b))
    assert (m.graph_replays == 5) == m.use_graphs
    # a slot that is used again starts from a zeroed state
    m.close_sequence(sa)
    sc = m.open_sequence()
    assert sc == sa
    got = m.step([StepEntry(sc, b, range(9))])
    assert np.abs(got.double().cpu().numpy() - plain(b)).max() < _tol(dtype, plain(b))


@pytest.mark.parametrize("dtype,sorts", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
def test_toy_feed_forward_with_routing(dtype, sorts, model_folders):
    """A feed-forward defined here that routes every token to one of two experts (router logits
    and the gate in float32, experts cut out of the dense weights) replaces layer 0's: registered,
    built and stepped with unequal prompts and then token by token.  The variant that gathers each
    expert's rows asks the device how many there are (a synchronisation) and says so
    (``capture_safe = False``); the other runs every expert on every row and masks, and is replayed
    inside the captured decode graphs of the bfloat16 path."""
    from dataclasses import replace
    from supersonic_b200.config.base import PartSpec
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.parts import register_feed_forward
    from supersonic_b200.weights import WeightStore

    @register_feed_forward("toy_top1")
    class ToyTop1:
        """logits = x Wr^T; e = argmax; out = softmax(logits)[e] * down_e(silu(gate_e x) * up_e x)."""

        capture_safe = not sorts

        def __init__(self, params, weights, build):
            self.n_experts = params["n_experts"]
            get = lambda k: build.weights.as_dtype(weights[k], torch.float32)
            self.gate, self.up, self.down = get("gate"), get("up"), get("down")
            self.router = self.gate[: self.n_experts]
            self.width = self.gate.shape[0] // self.n_experts

        def forward(self, ctx, x, residual):
            x = x.float()
            logits = x @ self.router.T
            prob = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            for e in range(self.n_experts):
                lo, hi = e * self.width, (e + 1) * self.width
                if not sorts:
                    g, u = x @ self.gate[lo:hi].T, x @ self.up[lo:hi].T
                    y = (torch.nn.functional.silu(g) * u) @ self.down[:, lo:hi].T
                    residual += torch.where((choice == e)[:, None], prob[:, e, None] * y, torch.zeros_like(y))
                    continue
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows]
                g, u = xe @ self.gate[lo:hi].T, xe @ self.up[lo:hi].T
                y = (torch.nn.functional.silu(g) * u) @ self.down[:, lo:hi].T
                residual[rows] += prob[rows, e, None] * y

    d, pc, pw = model_folders["C"]
    spec = _spec_with(tiny_configs.C)
    p0 = "model.layers.0.mlp"
    toy = PartSpec("toy_top1", {"n_experts": 2}, {"gate": f"{p0}.gate_proj.weight", "up": f"{p0}.up_proj.weight",
                                                  "down": f"{p0}.down_proj.weight"})
    spec = replace(spec, blocks=[replace(spec.blocks[0], feed_forward=toy)] + list(spec.blocks[1:]))
    m = Model(spec, WeightStore.from_dir(d), dtype=dtype, device=DEV, max_tokens=256)
    assert m.use_graphs == (dtype == "bfloat16" and not sorts)

    def plain(tokens):
        T = len(tokens)
        cos, sin = pl.rope_tables(pc, T)
        h = pl.embedding(tokens, pw["model.embed_tokens.weight"])
        h = h + pl.attention_mixer(pl.rms_norm(h, pw["model.layers.0.input_layernorm.weight"], pc["rms_norm_eps"]),
                                   pw, "model.layers.0", pc, cos, sin)
        x = pl.rms_norm(h, pw["model.layers.0.post_attention_layernorm.weight"], pc["rms_norm_eps"])
        gate, up, down = (pw[f"{p0}.{n}_proj.weight"] for n in ("gate", "up", "down"))
        width = gate.shape[0] // 2
        logits = x @ gate[:2].T
        prob = np.exp(logits - logits.max(-1, keepdims=True))
        prob /= prob.sum(-1, keepdims=True)
        out = np.zeros_like(h)
        used.update(int(e) for e in logits.argmax(-1))
        margins[tuple(tokens)] = (logits[:, 0] - logits[:, 1]).tolist()
        for t in range(T):
            e = int(logits[t].argmax())
            lo, hi = e * width, (e + 1) * width
            g, u = gate[lo:hi] @ x[t], up[lo:hi] @ x[t]
            out[t] = prob[t, e] * (down[:, lo:hi] @ (g / (1 + np.exp(-g)) * u))
        h = h + out
        for layer in range(1, pc["num_hidden_layers"]):
            h = pl.block(h, pw, layer, pc, cos, sin)
        return pl.output_head(h, pw, pc)

    used, margins = set(), {}
    rng = np.random.default_rng(8)
    a, b = rng.integers(0, 301, 23).tolist(), rng.integers(0, 301, 11).tolist()
    ra, rb = plain(a), plain(b)
    assert used == {0, 1}                                       # else the routing was not exercised
    sa, sb = m.open_sequence(), m.open_sequence()
    got = m.step([StepEntry(sa, a[:18], range(18)), StepEntry(sb, b[:6], range(6))])
    ga, gb = [got[:18]], [got[18:]]
    for i in range(5):
        got = m.step([StepEntry(sa, [a[18 + i]], [0]), StepEntry(sb, [b[6 + i]], [0])])
        ga.append(got[:1]); gb.append(got[1:])
    if dtype == "bfloat16":
        # a token whose two router logits are nearly equal may go to the other expert in bfloat16:
        # compare the rows whose choice is clear in the plain implementation
        clear = lambda toks: np.array([abs(m_) > 0.05 for m_ in margins[tuple(toks)]])
        ka, kb = clear(a), clear(b)
        assert ka.sum() >= 18 and kb.sum() >= 8
    else:
        ka, kb = np.ones(len(a), bool), np.ones(len(b), bool)
    assert np.abs(torch.cat(ga).double().cpu().numpy() - ra)[ka].max() < _tol(dtype, ra)
    assert np.abs(torch.cat(gb).double().cpu().numpy() - rb)[kb].max() < _tol(dtype, rb)
    assert (m.graph_replays == 5) == m.use_graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_encoding(dtype, model_folders):
    """A position encoding defined here (a learned vector per position added to every query and
    key head, no rotation) replaces the rotary one in every layer: registered, built, stepped; in
    bfloat16 beside the serving kernels, its decode steps inside the captured graphs."""
    from dataclasses import replace
    from supersonic_b200.cache import PAGE_SHIFT
    from supersonic_b200.config.base import PartSpec
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.parts import register_position_encoding
    from supersonic_b200.weights import WeightStore

    @register_position_encoding("toy_learned")
    class ToyLearned:
        def __init__(self, params, weights, build):
            self.head_dim = params["head_dim"]
            self.table = build.weights.as_dtype(weights["table"], torch.float32)[:, : self.head_dim].contiguous()

        def encode_and_append(self, ctx, qkv, kv, n_q, n_kv, write_cache=True):
            k_cache, v_cache, table, _ = kv
            n_rot = n_q + (n_kv if write_cache else 0)
            shift = 0.5 * self.table[ctx.batch.pos.long()]                       # [T, head_dim]
            heads = qkv[:, : n_rot * self.head_dim].view(qkv.shape[0], n_rot, self.head_dim)
            heads += shift[:, None, :].to(qkv.dtype)
            ctx.kernels.rope_append(qkv, None, None, ctx.batch, table, k_cache, v_cache, n_q, n_kv,
                                    self.head_dim, 0, PAGE_SHIFT, write_cache)

    d, pc, pw = model_folders["B"]
    spec = _spec_with(tiny_configs.B)
    toy = PartSpec("toy_learned", {"head_dim": pc["head_dim"]}, {"table": "model.embed_tokens.weight"})
    spec = replace(spec, blocks=[replace(b, position=toy) for b in spec.blocks])
    m = Model(spec, WeightStore.from_dir(d), dtype=dtype, device=DEV, max_tokens=256)
    assert m.use_graphs == (dtype == "bfloat16")

    def plain(tokens):
        T = len(tokens)
        nq, nkv, hd = pc["num_attention_heads"], pc["num_key_value_heads"], pc["head_dim"]
        shift = 0.5 * pw["model.embed_tokens.weight"][:T, :hd]
        h = pl.embedding(tokens, pw["model.embed_tokens.weight"])
        for layer in range(pc["num_hidden_layers"]):
            p = f"model.layers.{layer}"
            x = pl.rms_norm(h, pw[f"{p}.input_layernorm.weight"], pc["rms_norm_eps"])
            q = (x @ pw[f"{p}.self_attn.q_proj.weight"].T).reshape(T, nq, hd) + shift[:, None, :]
            k = (x @ pw[f"{p}.self_attn.k_proj.weight"].T).reshape(T, nkv, hd) + shift[:, None, :]
            v = (x @ pw[f"{p}.self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
            a = pl.attention_scores(q, k, v, 1 / math.sqrt(hd), None).reshape(T, nq * hd)
            h = h + a @ pw[f"{p}.self_attn.o_proj.weight"].T
            h = h + pl.swiglu_ffn(pl.rms_norm(h, pw[f"{p}.post_attention_layernorm.weight"], pc["rms_norm_eps"]), pw, p)
        return pl.output_head(h, pw, pc)

    toks = np.random.default_rng(9).integers(0, 384, 75).tolist()
    ref = plain(toks)
    s = m.open_sequence()
    got = [m.step([StepEntry(s, toks[:66], range(66))])]
    got += [m.step([StepEntry(s, [toks[p]], [0])]) for p in range(66, 75)]
    assert np.abs(torch.cat(got).double().cpu().numpy() - ref).max() < _tol(dtype, ref)
    assert m.graph_replays == (9 if dtype == "bfloat16" else 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_windowed_attention_through_the_engine(dtype, name, model_folders):
    """A window of 100 keys (no multiple of the page size) on every layer.  A prompt longer than the
    window runs in chunks of 48 tokens through the cache, decoding crosses a page edge, pages the
    window left behind go back and are taken by a second sequence whose own cached values are
    large, so that a read of a stale or recycled page would show."""
    from supersonic_b200.config.base import ScheduleEntry  # noqa: F401
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.weights import WeightStore
    d, pc, pw = model_folders[name]
    cfg = tiny_configs.CONFIGS[name][0]
    L = cfg["num_hidden_layers"]
    window = {i: 100 for i in range(L)}
    spec = _spec_with(cfg, None, window)
    m = Model(spec, WeightStore.from_dir(d), dtype=dtype, device=DEV, max_tokens=512, step_token_budget=48)
    order = [(i, i, True) for i in range(L)]
    rng = np.random.default_rng(31)
    a = rng.integers(0, pc["vocab_size"], 230).tolist()
    b = rng.integers(0, pc["vocab_size"], 150).tolist()
    ra, rb = (_plain_forward_scheduled(pc, pw, t, order, window) for t in (a, b))
    tol = lambda ref: 2e-5 if dtype == "float32" else 2e-2 * np.abs(ref).max()
    sa = m.open_sequence()
    got = [m.step([StepEntry(sa, a[:200], range(150, 200))])]          # five chunks; pages 0 and 1 are given back
    m.cache.check()
    group = m.cache.kv_groups[0]
    assert min(group.held[sa]) == 1 and group.need.window == 100
    free_after_a = group.pool.n_free
    sb = m.open_sequence()
    got_b = [m.step([StepEntry(sb, b[:120], range(100, 120))])]       # takes pages, among them what a gave back
    m.cache.check()
    for i in range(30):                                                 # both decode; a crosses the edge at 256? no: at 192+64
        rows = m.step([StepEntry(sa, [a[200 + i]], [0]), StepEntry(sb, [b[120 + i]], [0])])
        got.append(rows[:1]); got_b.append(rows[1:])
        m.cache.check()
    ga, gb = (torch.cat(g).double().cpu().numpy() for g in (got, got_b))
    assert np.abs(ga - ra[150:]).max() < tol(ra), "sequence a"
    assert np.abs(gb - rb[100:]).max() < tol(rb), "sequence b"
    assert group.pool.n_free <= free_after_a                             # b holds pages now
    m.close_sequence(sa)
    m.close_sequence(sb)
    m.cache.check()
    assert group.pool.n_held == 0


def test_a_wait_that_runs_out_inside_a_replayed_graph_is_reported(model_folders):
    """A decode step of the serving path is a graph replay: no Python launch wrapper runs.  A
    feed-forward defined here launches the probe whose only wait can never be satisfied (it gives
    up after about a second and sets the device's error word: no fault, no hang).  The error must be
    reported after the step that captured the graph and again after a step that only replayed it,
    and the logits of those steps (the probe touches no data) are right."""
    from dataclasses import replace
    from supersonic_b200.config.base import PartSpec
    from supersonic_b200.csrc import ops
    from supersonic_b200.engine import Model, StepEntry
    from supersonic_b200.parts import register_feed_forward
    from supersonic_b200.weights import WeightStore

    @register_feed_forward("toy_probe")
    class ToyProbe:
        def __init__(self, params, weights, build):
            self.device = build.device

        def forward(self, ctx, x, residual):
            ops.tc_wait_probe(self.device)

    d, pc, pw = model_folders["A"]
    spec = _spec_with(tiny_configs.A)
    spec = replace(spec, blocks=[spec.blocks[0], replace(spec.blocks[1], feed_forward=PartSpec("toy_probe", {}, {}))])
    m = Model(spec, WeightStore.from_dir(d), dtype="bfloat16", device=DEV, max_tokens=128)
    assert m.use_graphs
    ops.check_device_errors(DEV)                       # whatever earlier tests left is looked at and cleared
    toks = np.random.default_rng(41).integers(0, 256, 12).tolist()

    def plain(tokens):
        cos, sin = pl.rope_tables(pc, len(tokens))
        h = pl.block(pl.embedding(tokens, pw["model.embed_tokens.weight"]), pw, 0, pc, cos, sin)
        x = pl.rms_norm(h, pw["model.layers.1.input_layernorm.weight"], pc["rms_norm_eps"])
        return pl.output_head(h + pl.attention_mixer(x, pw, "model.layers.1", pc, cos, sin), pw, pc)

    ref = plain(toks)
    s = m.open_sequence()
    m.step([StepEntry(s, toks[:10], [])])
    with pytest.raises(ops.KernelError, match="bounded wait"):
        m.check_errors()
    m.check_errors()                                   # reported once
    first = m.step([StepEntry(s, [toks[10]], [0])])    # builds and captures the graph, then replays it
    with pytest.raises(ops.KernelError, match="bounded wait"):
        m.check_errors()
    replays = m.graph_replays
    second = m.step([StepEntry(s, [toks[11]], [0])])   # a replay and nothing else
    assert m.graph_replays == replays + 1
    with pytest.raises(ops.KernelError, match="bounded wait"):
        m.fetch(torch.zeros(1, dtype=torch.int32, device=DEV))
    m.check_errors()
    got = torch.cat([first, second]).double().cpu().numpy()
    assert np.abs(got - ref[10:]).max() < 2e-2 * np.abs(ref).max()
