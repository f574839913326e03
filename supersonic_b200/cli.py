"""Command line in the manner of the reference's ``supersonic`` binary
(crates/runner/src/main.rs:347-780): the same option names with the same meanings
where this library has them.  Prompts are token ids (``--prompt-ids``, ``--prompt-file``); a
text ``--prompt`` is accepted when the model folder has a ``tokenizer.json`` and the
``tokenizers`` package is installed, as the reference links the tokenizers crate
(crates/runner/src/llama31_engine.rs:871-880).  The model is a folder (``--model-dir``) or a
named size with random weights (``--preset`` with ``--random-seed``).  Output lines follow the
reference: ``[tokens] ...`` and the ``[..._json]`` lines on stdout, ``[vram]``, ``[weights]``,
``[prefill]``, ``[result]``, ``[stage]``, ``[teacher_forced]`` on stderr
(llama31_engine.rs:903-921, 1083-1087, 1564-1598, 432-463, 684-705).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="supersonic", description="SuperSonic-B200: LLM generation on one B200")
    ap.add_argument("--model", default=None,
                    help="model variant name (a preset's name); with --model-dir it is checked against the folder")
    ap.add_argument("--model-dir", default=None, help="model directory (config.json + safetensors)")
    ap.add_argument("--preset", default=None,
                    help="a named size (see --list-presets) built with random weights instead of a folder")
    ap.add_argument("--random-seed", type=int, default=0, help="seed of the random weights of --preset")
    ap.add_argument("--list-presets", action="store_true", help="print the preset names and exit")
    ap.add_argument("--prompt", default="", help="text prompt (needs tokenizer.json)")
    ap.add_argument("--prompt-no-special-tokens", action="store_true",
                    help="do not add tokenizer special tokens when encoding --prompt")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="comma-separated token ids; repeat for a batch of prompts")
    ap.add_argument("--prompt-file", action="append", default=[],
                    help="a file with one prompt a line, token ids separated by commas or spaces ('#' starts a comment)")
    ap.add_argument("--max-new-tokens", type=int, default=8, help="maximum tokens to generate")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy argmax")
    ap.add_argument("--top-k", type=int, default=0, help="keep the K most probable tokens; 0 = no cap")
    ap.add_argument("--top-p", type=float, default=1.0, help="nucleus mass; 1.0 = no truncation")
    ap.add_argument("--sampling-seed", type=int, default=42, help="seed for non-greedy sampling")
    ap.add_argument("--stop-ids", default=None,
                    help="comma-separated token ids that end a sequence (default: the model's eos_token_id)")
    ap.add_argument("--context-size", type=int, default=None,
                    help="maximum context in tokens (prompt + generated); sizes the cache")
    ap.add_argument("--backend", default="auto", help="'auto' or 'cuda' (the only backend)")
    ap.add_argument("--device", type=int, default=0, help="CUDA device ordinal")
    ap.add_argument("--batch-size", type=int, default=1, help="sequences decoded in parallel")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="bfloat16 (serving kernels) or float32 (true 32-bit path)")
    ap.add_argument("--emit-stage-timings", action="store_true",
                    help="print [stage] lines: device time by stage (projections, attention, mlp, norms, head, sampling)")
    ap.add_argument("--emit-generated-json", action="store_true",
                    help="print [generated_json] with the generated ids (and text, with a tokenizer)")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at stop tokens")
    ap.add_argument("--teacher-forced", action="store_true",
                    help="score the prompts with teacher forcing instead of generating new tokens")
    ap.add_argument("--teacher-forced-decode-step", action="store_true",
                    help="with --teacher-forced: one token as the prompt, then one decode step per token")
    return ap


def parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def read_prompt_file(path: str) -> List[List[int]]:
    prompts = []
    with open(path, "r", encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            line = line.split("#", 1)[0].strip()
            if not line:
                continue
            try:
                prompts.append(parse_ids(line))
            except ValueError:
                raise ValueError(f"{path}:{n}: token ids must be integers") from None
    return prompts


def _tokenizer(model_dir):
    if not model_dir:
        return None
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    err = lambda msg: print(msg, file=sys.stderr)
    from .config import ConfigError, load_config, preset_names
    if args.list_presets:
        print("\n".join(preset_names()))
        return 0
    if args.backend not in ("auto", "cuda"):
        err(f"backend {args.backend!r} is not available: this build is CUDA sm_100a only")
        return 2
    preset = args.preset
    if not args.model_dir and not preset and args.model:
        preset = args.model.lower().replace("_", "-")           # --model NAME alone: that size, random weights
    if bool(args.model_dir) == bool(preset):
        err("give --model-dir DIR, or --preset NAME [--random-seed S] (names: " + ", ".join(preset_names()) + ")")
        return 2
    if preset and preset not in preset_names():
        err(f"unknown preset {preset!r}; known: {', '.join(preset_names())}")
        return 2
    if args.model_dir and args.model:
        cfg = load_config(args.model_dir)
        name = args.model.lower().replace("_", "-")
        if name not in preset_names() and name != cfg.model_type:
            err(f"[warn] --model {args.model} is not a name this build knows; the folder's "
                f"architecture {cfg.architectures[0]} decides")
    tok = _tokenizer(args.model_dir)
    try:
        prompts = [parse_ids(p) for p in args.prompt_ids]
        for path in args.prompt_file:
            prompts += read_prompt_file(path)
        stop_ids = parse_ids(args.stop_ids) if args.stop_ids is not None else None
    except (ValueError, OSError) as e:
        err(str(e))
        return 2
    if args.prompt:
        if tok is None:
            err("--prompt needs tokenizer.json in the model folder and the tokenizers package; use --prompt-ids")
            return 2
        prompts.append(tok.encode(args.prompt, add_special_tokens=not args.prompt_no_special_tokens).ids)
    if not prompts or any(not p for p in prompts):
        err("give --prompt-ids 1,2,3 (repeatable), --prompt-file FILE or --prompt TEXT; no prompt may be empty")
        return 2
    new_tokens = 0 if args.teacher_forced else args.max_new_tokens
    longest = max(len(p) for p in prompts)
    context = args.context_size or (longest + new_tokens)
    if context < longest + new_tokens:
        err(f"--context-size {context} < prompt_tokens {longest} + max_new_tokens {new_tokens}")
        return 2
    batch = max(args.batch_size, 1)
    from .api import load
    from .engine.preflight import MemoryPreflightError
    t0 = time.time()
    try:
        engine = load(args.model_dir, dtype=args.dtype, device=args.device, context_size=context,
                      batch_size=min(batch, len(prompts)), preset=preset, random_seed=args.random_seed)
    except (MemoryPreflightError, ConfigError) as e:
        err(str(e))
        return 1
    model = engine.model
    err(model.memory_estimate.line(model.cache.n_pages * 64))
    err(f"[weights] loaded in {(time.time() - t0) * 1e3:.0f}ms")

    if args.teacher_forced:
        return _teacher_forced(args, engine, prompts, batch)

    from .sampling import SamplingParams
    gen = engine.generator
    if args.emit_stage_timings:
        gen.time_stages(True)
    results = gen.generate(
        prompts, args.max_new_tokens,
        SamplingParams(args.temperature, args.top_k, args.top_p, args.sampling_seed),
        stop_token_ids=stop_ids, ignore_eos=args.ignore_eos, batch_size=batch)
    st = gen.stats
    err(f"[prefill] {st.prefill_tokens} tokens in {st.prefill_s * 1e3:.0f}ms ({st.prefill_steps} batch"
        f"{'es' if st.prefill_steps != 1 else ''})")
    for p, r in zip(prompts, results):
        if tok is not None:
            print(tok.decode(list(p) + r.tokens, skip_special_tokens=True))
        if args.emit_generated_json:
            payload = {"generated_ids": r.tokens, "finish_reason": r.finish_reason}
            if tok is not None:
                payload["generated_text"] = tok.decode(r.tokens, skip_special_tokens=True)
            print("[generated_json] " + json.dumps(payload))
        print("[tokens] " + " ".join(str(t) for t in r.tokens))
    n_gen = sum(len(r.tokens) for r in results)
    err(f"[result] prompt_tokens={sum(len(p) for p in prompts)} generated_tokens={n_gen} "
        f"decode_ms={st.decode_s * 1e3:.0f} ms_per_step={st.decode_s * 1e3 / max(st.decode_steps, 1):.1f}")
    if args.emit_stage_timings:
        err(gen.stage_timings["prefill"].line("prefill"))
        err(gen.stage_timings["decode"].line("decode"))
    return 0


def _teacher_forced(args, engine, prompts, batch) -> int:
    from .engine.score import teacher_forced
    if any(len(p) < 2 for p in prompts):
        print("--teacher-forced requires at least 2 prompt tokens", file=sys.stderr)
        return 2
    for lo in range(0, len(prompts), batch):
        for sc in teacher_forced(engine.model, prompts[lo:lo + batch], decode_step=args.teacher_forced_decode_step):
            d = sc.to_dict()
            print(f"[teacher_forced] tokens={sc.tokens} scored_tokens={sc.scored_tokens} decode_steps={sc.decode_steps} "
                  f"nll={sc.total_nll:.6f} avg_nll={sc.avg_nll:.6f} ppl={sc.perplexity:.6f} bpt={sc.bits_per_token:.6f} "
                  f"total_ms={sc.total_ms:.1f} ms_per_token={d['ms_per_token']:.2f}", file=sys.stderr)
            d.update(backend="cuda", mode="dense", model=args.model or args.preset or "",
                     teacher_forced_scoring="decode_step_logits" if args.teacher_forced_decode_step
                     else "prompt_step_target_nll")
            print("[teacher_forced_json] " + json.dumps(d))
    return 0


if __name__ == "__main__":
    sys.exit(main())
