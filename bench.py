"""Benchmark: decode tokens per second of a Llama-3.1-8B-sized model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

One JSON line on stdout.  ``value`` is decoded tokens per second at batch 8 (one step = one
decode step of the whole batch and the greedy pick of its tokens, timed on the device with CUDA
events around exactly K steps after W warm-up steps).  ``e2e`` is the same through the Python
entry point (``Engine.generate``): host token lists in, host token lists out, every step copying
its token ids from pinned host memory and reading the sampled tokens back.  ``prefill`` is one
2,048-token prompt; ``points`` holds decode at batch 1 and 64 and the two further workloads the
benchmark definition lists (a ragged batch of 16 prompts at Llama-3.2-3B sizes, a ragged batch of
64 prompts sampled at temperature 1.0 at Llama-3.2-1B sizes), each through the entry point;
``stages`` is the device time of one uncaptured decode step and one prompt step by stage;
``roofline`` is the decode step's bytes (every weight the built model's parts hold, once, plus the
live sequences' keys and values) over its time.  Weights are ~15 GB, far beyond the 126 MB L2, so
no flush is needed between steps.

``--impl reference``: the reference is a Rust workspace that cannot be built here, so the whole
engine is ``unavailable``; its CUDA kernels do build (``baseline/reference_kernels.py``), and the
line carries their times per operation at the same shapes under ``reference_ops``.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out, src = dict(FALLBACK_PEAKS), "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
        for k in out:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
                src = "measured"
    except (OSError, ValueError):
        pass
    return out, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.samples, self.proc, self.device = [], None, device

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append(parts)

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm = sorted(int(s[0]) for s in self.samples)
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(self.samples[0][1]) if self.samples else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def prefill_flops(model, lengths, wanted_rows):
    """FLOPs of a prompt step: 2 per weight element per token for every matrix the model's parts
    hold (asked of the built model), causal attention (QK and PV) for the mixers that say how many
    query heads of which size they have, and the head for the wanted rows."""
    tokens = sum(lengths)
    linear = 2 * tokens * model.matrix_elements()
    attn = 0
    for stop in model.spec.schedule:
        mixer = model.blocks[stop.layer].mixer
        n_q, hd = getattr(mixer, "n_q", 0), getattr(mixer, "head_dim", 0)
        attn += sum(2 * 2 * n_q * hd * n * (n + 1) / 2 for n in lengths)
    return linear + attn + 2 * wanted_rows * model.spec.vocab_size * model.spec.hidden_size


def time_decode(model, batch, prompt_len, steps, warmup, seed=0):
    """(ms per step, kernels per step, bytes a step reads at the middle of the timed region) of decode
    at ``batch`` sequences after prompts of ``prompt_len``.  A step is the model's decode step plus
    the greedy pick of every sequence's token from its logits, all on the device; the tokens fed
    are given (the pick is not read back: that is what ``e2e`` adds)."""
    import torch
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.sampling import Sampler, SamplingParams
    g = torch.Generator().manual_seed(seed)
    slots = [model.open_sequence() for _ in range(batch)]
    sampler, greedy = Sampler(model.kernels, model.cache.rng_state), SamplingParams()
    slot_t = torch.tensor(slots, dtype=torch.int32, device=model.device)
    try:
        prompts = torch.randint(0, model.vocab_size, (batch, prompt_len), generator=g).tolist()
        for lo in range(0, batch, 8):                     # prompts in groups: bounded activation memory
            model.step([StepEntry(s, p, []) for s, p in zip(slots[lo:lo + 8], prompts[lo:lo + 8])])
        nxt = torch.randint(0, model.vocab_size, (warmup + steps, batch), generator=g).tolist()
        for w in range(warmup):
            sampler(model.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt[w])]), slot_t, greedy)
        torch.cuda.synchronize()
        k0 = model.graph_kernels
        bytes_first = model.decode_step_bytes(slots)              # host arithmetic, outside the timed region
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(steps):
            sampler(model.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt[warmup + k])]), slot_t, greedy)
        end.record()
        torch.cuda.synchronize()
        model.check_errors()
        bytes_mid = (bytes_first + model.decode_step_bytes(slots)) // 2     # the cache grows by a token a step
        return start.elapsed_time(end) / steps, (model.graph_kernels - k0) // max(steps, 1) + 1, bytes_mid
    finally:
        for s in slots:
            model.close_sequence(s)


def stage_shares(model, batch, prompt_len, prefill_tokens, seed=5):
    """Device milliseconds by stage of one uncaptured decode step of ``batch`` sequences and of one
    prompt step (see supersonic_b200/engine/stage_timings.py)."""
    import torch
    from supersonic_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    slots = [model.open_sequence() for _ in range(batch)]
    out = {}
    try:
        prompts = torch.randint(0, model.vocab_size, (batch, prompt_len), generator=g).tolist()
        model.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
        model.time_stages(True)
        for rep in range(2):                                   # the first timed step warms the uncaptured path
            model.step([StepEntry(s, [1], [0]) for s in slots])
            out["decode"] = {k: round(v, 4) for k, v in model.stage_times().items() if v > 0}
        model.close_sequence(slots.pop())
        for rep in range(2):
            s = model.open_sequence()
            model.step([StepEntry(s, torch.randint(0, model.vocab_size, (prefill_tokens,), generator=g).tolist(),
                                  [prefill_tokens - 1])])
            out["prefill"] = {k: round(v, 3) for k, v in model.stage_times().items() if v > 0}
            model.close_sequence(s)
    finally:
        model.time_stages(False)
        for s in slots:
            model.close_sequence(s)
    return out


def ragged_workload(preset, n_prompts, lo, hi, new_tokens, temperature, pk, seed):
    """A further workload of the benchmark definition through the Python entry point: ``n_prompts``
    prompts with lengths uniform in [lo, hi] start together (one prompt step, in chunks of the step's
    token budget), then ``new_tokens`` decode steps.  Host wall time from a step's start to its tokens
    on the host; the decode fraction uses the bytes at the middle of the run."""
    import torch
    import supersonic_b200
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(lo, hi + 1, (n_prompts,), generator=g).tolist()
    ctx = -(-(max(lengths) + new_tokens) // 64) * 64
    eng = supersonic_b200.load(preset=preset, random_seed=seed, context_size=ctx, batch_size=n_prompts,
                               max_tokens=sum(-(-(n + new_tokens) // 64) * 64 for n in lengths))
    model = eng.model
    prompts = [torch.randint(0, model.vocab_size, (n,), generator=g).tolist() for n in lengths]
    # once untimed: decode steps replay one captured graph per (batch size, context bucket), and capturing
    # them (a tenth of a second each) is a cost of a server's first minutes, not of a step
    eng.generate(prompts, max_new_tokens=new_tokens, temperature=temperature, ignore_eos=True, batch_size=n_prompts)
    eng.generator.stats = type(eng.generator.stats)()
    eng.generate(prompts, max_new_tokens=new_tokens, temperature=temperature, ignore_eos=True, batch_size=n_prompts)
    st = eng.generator.stats
    mid = [n + new_tokens // 2 for n in lengths]
    item = 2
    kv_mid = sum(model.cache.kv_groups[0].need.n_kv_heads * model.cache.kv_groups[0].need.head_dim * 2 * item
                 * len(model.cache.kv_groups[0].entries) * n for n in mid)
    step_bytes = model.weight_bytes() + kv_mid
    decode_ms = st.decode_s * 1e3 / max(st.decode_steps, 1)
    out = {"prompts": n_prompts, "prompt_tokens": sum(lengths), "new_tokens": new_tokens,
           "prefill_tok_s": round(st.prefill_tokens / st.prefill_s, 1),
           "prefill_frac": round(prefill_flops(model, lengths, n_prompts) / st.prefill_s / (pk["bf16_tflops"] * 1e12), 4),
           "decode_tok_s": round(st.decode_tokens / st.decode_s, 1), "decode_ms_per_step": round(decode_ms, 4),
           "decode_hbm_frac": round(step_bytes / (decode_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
           "temperature": temperature}
    del eng, model
    torch.cuda.empty_cache()
    return out


def time_prefill(model, tokens, reps=5, warmup=3, seed=1, seqs=1):
    """Best device time of one step that brings ``seqs`` prompts of ``tokens`` tokens each (new random
    tokens every time; the wanted row is each prompt's last).  The first runs are warm-up; a step whose
    sizes recur replays a captured graph from its second run on, as it would when serving."""
    import torch
    from supersonic_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    best = None
    for r in range(reps + warmup):
        prompts = torch.randint(0, model.vocab_size, (seqs, tokens), generator=g).tolist()
        slots = [model.open_sequence() for _ in range(seqs)]
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        model.step([StepEntry(s, p, [tokens - 1]) for s, p in zip(slots, prompts)])
        end.record()
        torch.cuda.synchronize()
        for s in slots:
            model.close_sequence(s)
        if r >= warmup:
            ms = start.elapsed_time(end)
            best = ms if best is None else min(best, ms)
    return best


def sweep(model, pk, steps, warmup):
    """Decode at further batch sizes and context lengths, prompts of further sizes: the table of README.md."""
    out = {"decode": [], "prefill": []}
    sizes = [(1, 512), (1, 8000), (8, 512), (8, 8000), (32, 512), (64, 512), (64, 4096)]
    if model.cache.max_seq_tokens >= 131072:               # --context 131072 --slots 4: the position limit too
        sizes.insert(2, (1, 131000))
    for batch, ctx in sizes:
        ms, _, nbytes = time_decode(model, batch, ctx, min(steps, 48), warmup, seed=20 + batch)
        out["decode"].append({"batch": batch, "context": ctx, "ms_per_step": round(ms, 3),
                              "tokens_s": round(batch * 1000.0 / ms, 1),
                              "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)})
    for seqs, tokens in ((1, 128), (1, 512), (1, 2048), (1, 8192), (8, 512), (4, 2048), (16, 128)):
        ms = time_prefill(model, tokens, reps=4, warmup=3, seed=30 + seqs, seqs=seqs)
        flops = prefill_flops(model, [tokens] * seqs, seqs)
        out["prefill"].append({"seqs": seqs, "tokens": tokens, "ms": round(ms, 3),
                               "tokens_s": round(seqs * tokens * 1000.0 / ms, 1),
                               "bf16_frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3)})
    return out


def time_e2e(engine, batch, prompt_len, steps, warmup, seed=2):
    """Decoded tokens per second through Engine.generate, host lists in and out."""
    import torch
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, engine.model.vocab_size, (batch, prompt_len), generator=g).tolist()
    stamps = []

    def on_step(live, tokens):                             # tokens are on the host when this runs
        stamps.append(time.perf_counter())
    from supersonic_b200.sampling import SamplingParams
    engine.generator.generate(prompts, max_new_tokens=warmup + steps + 1, sampling=SamplingParams(),
                              ignore_eos=True, batch_size=batch, on_step=on_step)
    # stamps[0] follows the prompt step; stamps[i] follows decode step i
    dt = stamps[warmup + steps] - stamps[warmup]
    return batch * steps / dt


def reference_arm(args):
    """The reference's whole engine cannot run here (Rust, no cargo in the image).  Its CUDA kernels
    can: compiled unmodified for sm_100a, the ones its Llama lane uses are timed per operation at the
    shapes of this benchmark (the harness the reference times its engine with is
    tests/sm86/bench_llama31_8b.sh:31-175).  These figures explain; they are not an engine rate."""
    line = {"impl": "reference",
            "unavailable": "DeanoC/SuperSonic is a Rust workspace (Cargo.toml only, no setup.py or pyproject.toml): "
                           "pip cannot install it and no cargo/rustc is in the image; only its CUDA kernels are timed"}
    try:
        line["reference_ops"] = time_reference_ops(args)
    except Exception as e:      # noqa: BLE001 - the arm must print its line whatever happens
        line["reference_ops_unavailable"] = f"{type(e).__name__}: {str(e)[:200]}"
    print(json.dumps(line))
    return 0


def time_reference_ops(args):
    import torch
    from baseline import reference_kernels as rk
    from supersonic_b200.config import preset_config
    why = rk.available()
    if why:
        try:
            rk.install()
        except rk.ReferenceUnavailable as e:
            raise RuntimeError(f"{why}; {e}") from None
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device")
    cfg = preset_config(args.preset)
    dev = "cuda:0"
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    T, L = args.prefill_tokens, cfg.num_hidden_layers
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.05).to(torch.bfloat16)

    def timed(fn, reps=3):
        fn()                                                    # warm-up (the launchers synchronise)
        best = None
        for _ in range(reps):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
        return round(best, 4)

    ops = {}
    x = rnd(T, H)
    shapes = {"q": (nq * hd, H), "k": (nkv * hd, H), "v": (nkv * hd, H), "o": (H, nq * hd),
              "gate": (I, H), "up": (I, H), "down": (H, I)}
    weights = {n: rnd(*s) for n, s in shapes.items()}
    # K3: the tiled prompt GEMM (kernels/full_attention_4b_cuda.cuh:2671-2743), M = prompt tokens
    for n, w in weights.items():
        a = x if w.shape[1] == H else rnd(T, w.shape[1])
        ops[f"prefill_gemm_{n}_ms"] = timed(lambda a=a, w=w: rk.matmul_rhs_transposed(a, w), reps=2)
    # K6: prompt attention, one warp a query row (kernels/full_attention_cuda.cuh:360-474)
    q, k, v = rnd(1, nq, T, hd), rnd(1, nkv, T, hd), rnd(1, nkv, T, hd)
    ops["prefill_attention_ms"] = timed(lambda: rk.attention_prefill(q, k, v, hd ** -0.5), reps=1)
    # K2: RMSNorm over the prompt's rows and over one row
    wn = rnd(H)
    ops["prefill_rms_norm_ms"] = timed(lambda: rk.rms_norm(x, wn, 1e-5))
    x1 = rnd(1, H)
    ops["decode_rms_norm_ms"] = timed(lambda: rk.rms_norm(x1, wn, 1e-5))
    # K11: the decode projections, one row through cuBLAS (kernels/full_attention_bridge_4b_cuda.cu:4768-4813)
    for n, w in weights.items():
        a = rnd(w.shape[1])
        ops[f"decode_gemv_{n}_ms"] = timed(lambda a=a, w=w: rk.gemv_bf16(a, w))
    head = rnd(V, H)
    ops["decode_lm_head_ms"] = timed(lambda: rk.gemv_bf16(x1[0], head))
    ops["decode_lm_head_argmax_ms"] = timed(lambda: rk.lm_head_argmax(x1[0], head))
    # K13: decode attention of one sequence at the benchmark's mean context (kernels/full_attention_cuda.cuh:578-679)
    ctx = args.prompt_len + 128
    q1, kc, vc = rnd(1, nq, hd), rnd(1, nkv, 8192, hd), rnd(1, nkv, 8192, hd)
    ops["decode_attention_ms"] = timed(lambda: rk.attention_decode(q1, kc, vc, hd ** -0.5, kv_len=ctx))
    gate1, up1 = rnd(I), rnd(I)
    ops["decode_swiglu_ms"] = timed(lambda: rk.swiglu_mul(gate1, up1))
    layer = sum(ops[f"decode_gemv_{n}_ms"] for n in shapes) + ops["decode_attention_ms"] \
        + 2 * ops["decode_rms_norm_ms"] + ops["decode_swiglu_ms"]
    ops["decode_step_kernel_sum_ms"] = round(L * layer + ops["decode_rms_norm_ms"] + ops["decode_lm_head_ms"], 3)
    pre = sum(ops[f"prefill_gemm_{n}_ms"] for n in shapes) + ops["prefill_attention_ms"] + 2 * ops["prefill_rms_norm_ms"]
    ops["prefill_kernel_sum_ms"] = round(L * pre, 1)
    ops["note"] = ("per-operation device times of the reference's own kernels at these shapes (batch 1, "
                   f"{T}-token prompt, context {ctx}); the sums count one launch per operation and layer and "
                   "leave out rope, appends, residual adds and every host step of the reference's engine")
    return ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="llama3.1-8b")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the preset has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--context", type=int, default=8192, help="tokens per cache slot")
    ap.add_argument("--slots", type=int, default=64)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    ap.add_argument("--skip-workloads", action="store_true", help="leave out the 3B and 1B ragged workloads")
    ap.add_argument("--sweep", action="store_true",
                    help="also time decode and prompts at further sizes (adds a 'sweep' key to the line)")
    ap.add_argument("--deterministic", action="store_true",
                    help="time the bfloat16 path without float atomics and with one kernel choice whatever the batch")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this library has no multi-GPU path); got --gpus {args.gpus}")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from supersonic_b200.api import Engine
    from supersonic_b200.config import preset_config
    from supersonic_b200.csrc import ops
    from supersonic_b200.engine import Model
    from supersonic_b200.weights import RandomWeightStore

    full = preset_config(args.preset)
    layers = args.layers or full.num_hidden_layers
    cfg = preset_config(args.preset, num_hidden_layers=layers)
    pk, pk_src = peaks()
    t0 = time.time()
    store = RandomWeightStore(cfg, seed=2, device="cuda:0", std=0.02, norm_jitter=0.0)
    model = Model.from_config(cfg, store, dtype="bfloat16", device="cuda:0",
                              max_tokens=args.slots * args.context, max_seq_tokens=args.context,
                              deterministic=args.deterministic)
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t0:.1f} s, "
          f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device", file=sys.stderr)

    clocks = ClockSampler()
    clocks.start()
    launches0 = ops.LAUNCHES
    ms, kernels_per_step, bytes_step = time_decode(model, args.batch, args.prompt_len, args.steps, args.warmup)
    value = args.batch * 1000.0 / ms
    achieved = bytes_step / (ms * 1e-3) / 1e9

    engine = Engine(model)
    # On a device that has been under load, the decode steps right after a batch's prompts run slower
    # for some 60 ms, in plateaus (measured per step through Engine.generate: 3.33, then 3.03, then
    # 2.92 ms from the 23rd step on; a device that was idle before shows 2.90 ms from the first step):
    # the part's power management after the prompts' burst of tensor work, whether the prompts ran as a
    # captured graph or launch by launch.  The end-to-end figure is the steady rate, like the device-timed
    # one: it skips at least 24 steps before it times K, and says so in the record.
    e2e_warmup = max(args.warmup, 24)
    e2e = time_e2e(engine, args.batch, args.prompt_len, args.steps, e2e_warmup)

    pf_ms = time_prefill(model, args.prefill_tokens)
    pf_flops = prefill_flops(model, [args.prefill_tokens], 1)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, _, pbytes = time_decode(model, b, args.prompt_len, min(args.steps, 64), args.warmup, seed=10 + b)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
            points[f"decode_b{b}_hbm_frac"] = round(pbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
    stages = stage_shares(model, args.batch, args.prompt_len, args.prefill_tokens)
    swept = sweep(model, pk, args.steps, args.warmup) if args.sweep else None
    if not args.skip_workloads and layers == full.num_hidden_layers:
        del engine, model, store
        torch.cuda.empty_cache()
        # the benchmark definition's two further workloads: 16 prompts of 64..2,048 tokens then 128 steps at
        # Llama-3.2-3B sizes; 64 prompts of 1..4,096 tokens then 512 steps at temperature 1.0 at 1B sizes
        points["llama3.2-3b_ragged16"] = ragged_workload("llama3.2-3b", 16, 64, 2048, 128, 0.0, pk, seed=3)
        points["llama3.2-1b_ragged64"] = ragged_workload("llama3.2-1b", 64, 1, 4096, 512, 1.0, pk, seed=4)
    clk = clocks.stop()

    line = {
        "metric": "decode tokens/s at batch 8 (Llama 3.1 8B sizes, random bf16 weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 2, N(0, 0.02), norms 1), uniform random token ids",
        "impl": "ours",
        "config": {"model": args.preset, "layers": layers, "layers_full": full.num_hidden_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": args.prompt_len, "context_per_slot": args.context,
                   "slots": args.slots, "prefill_tokens": args.prefill_tokens, "parallelism": "none",
                   "l2": "inputs exceed L2 (15 GB of weights per step)", "peaks": pk_src,
                   "deterministic": bool(args.deterministic)},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * 4 * args.batch,
                "d2h_bytes_per_step": 4 * args.batch, "warmup": e2e_warmup,
                "note": "positions and slots go up every step, sampled tokens come back; the step's tokens stay on the device; the steps right after the prompts (slower for about 60 ms on a loaded device) are warm-up"},
        "gpu_launches": kernels_per_step * args.steps,
        "kernels_per_step": kernels_per_step,
        "step": "decode step of the batch + greedy pick on the device",
        "prefill": {"value": round(args.prefill_tokens * 1000.0 / pf_ms, 1), "tokens": args.prefill_tokens,
                    "ms": round(pf_ms, 3), "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "stages": stages,
        **({"sweep": swept} if swept else {}),
        "clocks": clk,
    }
    assert ops.LAUNCHES > launches0
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
