"""Benchmark: decode tokens per second of a Llama-3.1-8B-sized model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

One JSON line on stdout.  ``value`` is decoded tokens per second at batch 8 (one step = one
decode step of the whole batch, timed on the device with CUDA events around exactly K graph
replays after W warm-up steps).  ``e2e`` is the same through the Python entry point
(``Engine.generate``): host token lists in, host token lists out, every step copying its
token ids from pinned host memory and reading the sampled tokens back.  ``prefill`` is one
2,048-token prompt; ``points`` holds decode at batch 1 and 64; ``roofline`` is the decode
step's bytes (every weight once plus the live sequences' keys and values) over its time.
Weights are ~15 GB, far beyond the 126 MB L2, so no flush is needed between steps.
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


def decode_bytes(cfg, layers, batch, context, dtype_bytes=2):
    """Bytes a decode step must read: each used weight once (embedding rows aside) and the
    keys and values of the live sequences."""
    h, i = cfg.hidden_size, cfg.intermediate_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = h * q + 2 * h * kv + q * h + 3 * h * i + 2 * h
    weights = (layers * per_layer + h + cfg.vocab_size * h) * dtype_bytes
    kv_bytes = layers * 2 * kv * dtype_bytes * context * batch
    return weights + kv_bytes


def prefill_flops(cfg, layers, tokens):
    h, i = cfg.hidden_size, cfg.intermediate_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    linear = 2 * tokens * (h * q + 2 * h * kv + q * h + 3 * h * i)
    attn = 2 * 2 * cfg.num_attention_heads * cfg.head_dim * tokens * (tokens + 1) / 2      # causal QK and PV
    return layers * (linear + attn) + 2 * cfg.vocab_size * h                              # one row of logits


def time_decode(model, batch, prompt_len, steps, warmup, seed=0):
    """(ms per step, kernels per step) of decode at ``batch`` sequences after prompts of ``prompt_len``."""
    import torch
    from supersonic_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    slots = [model.open_sequence() for _ in range(batch)]
    try:
        prompts = torch.randint(0, model.vocab_size, (batch, prompt_len), generator=g).tolist()
        for lo in range(0, batch, 8):                     # prompts in groups: bounded activation memory
            model.step([StepEntry(s, p, []) for s, p in zip(slots[lo:lo + 8], prompts[lo:lo + 8])])
        nxt = torch.randint(0, model.vocab_size, (warmup + steps, batch), generator=g).tolist()
        for w in range(warmup):
            model.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt[w])])
        torch.cuda.synchronize()
        k0 = model.graph_kernels
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(steps):
            model.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt[warmup + k])])
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / steps, (model.graph_kernels - k0) // max(steps, 1)
    finally:
        for s in slots:
            model.close_sequence(s)


def time_prefill(model, tokens, reps=5, warmup=3, seed=1):
    import torch
    from supersonic_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    best = None
    for r in range(reps + warmup):
        prompt = torch.randint(0, model.vocab_size, (tokens,), generator=g).tolist()
        slot = model.open_sequence()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        model.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        model.close_sequence(slot)
        if r >= warmup:                                    # the first runs are warm-up
            ms = start.elapsed_time(end)
            best = ms if best is None else min(best, ms)
    return best


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
    ap.add_argument("--skip-points", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "DeanoC/SuperSonic is a Rust workspace (Cargo.toml only, no setup.py or "
                          "pyproject.toml): pip cannot install it and no cargo/rustc is in the image"}))
        return 0
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
                              max_tokens=args.slots * args.context, max_seq_tokens=args.context)
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t0:.1f} s, "
          f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device", file=sys.stderr)

    clocks = ClockSampler()
    clocks.start()
    launches0 = ops.LAUNCHES
    ms, kernels_per_step = time_decode(model, args.batch, args.prompt_len, args.steps, args.warmup)
    ctx_mid = args.prompt_len + args.warmup + args.steps / 2
    value = args.batch * 1000.0 / ms
    bytes_step = decode_bytes(cfg, layers, args.batch, ctx_mid)
    achieved = bytes_step / (ms * 1e-3) / 1e9

    engine = Engine(model)
    e2e = time_e2e(engine, args.batch, args.prompt_len, args.steps, args.warmup)

    pf_ms = time_prefill(model, args.prefill_tokens)
    pf_flops = prefill_flops(cfg, layers, args.prefill_tokens)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, _ = time_decode(model, b, args.prompt_len, min(args.steps, 64), args.warmup, seed=10 + b)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
            points[f"decode_b{b}_hbm_frac"] = round(
                decode_bytes(cfg, layers, b, args.prompt_len + args.warmup + min(args.steps, 64) / 2)
                / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
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
                   "l2": "inputs exceed L2 (15 GB of weights per step)", "peaks": pk_src},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 3 * 4 * args.batch,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": kernels_per_step * args.steps,
        "kernels_per_step": kernels_per_step,
        "prefill": {"value": round(args.prefill_tokens * 1000.0 / pf_ms, 1), "tokens": args.prefill_tokens,
                    "ms": round(pf_ms, 3), "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clk,
    }
    assert ops.LAUNCHES > launches0
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
