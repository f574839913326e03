"""Command line in the manner of the reference's ``supersonic`` binary
(crates/runner/src/main.rs:347-780): the same option names with the same meanings
where this library has them.  Prompts are token ids (``--prompt-ids``); a text
``--prompt`` is accepted when the model folder has a ``tokenizer.json`` and the
``tokenizers`` package is installed, as the reference links the tokenizers crate
(crates/runner/src/llama31_engine.rs:871-880).  Output lines follow the reference:
``[tokens] ...`` on stdout, ``[prefill]``/``[result]`` on stderr
(llama31_engine.rs:1083-1087, 1564-1598).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="supersonic", description="SuperSonic-B200: LLM generation on one B200")
    ap.add_argument("--model", default=None,
                    help="model variant name; checked against the folder's architecture if given")
    ap.add_argument("--model-dir", required=True,
                    help="model directory (config.json + safetensors)")
    ap.add_argument("--prompt", default="", help="text prompt (needs tokenizer.json)")
    ap.add_argument("--prompt-no-special-tokens", action="store_true",
                    help="do not add tokenizer special tokens when encoding --prompt")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="comma-separated token ids; repeat for a batch of prompts")
    ap.add_argument("--max-new-tokens", type=int, default=8, help="maximum tokens to generate")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy argmax")
    ap.add_argument("--top-k", type=int, default=0, help="keep the K most probable tokens; 0 = no cap")
    ap.add_argument("--top-p", type=float, default=1.0, help="nucleus mass; 1.0 = no truncation")
    ap.add_argument("--sampling-seed", type=int, default=42, help="seed for non-greedy sampling")
    ap.add_argument("--context-size", type=int, default=None,
                    help="maximum context in tokens (prompt + generated); sizes the cache")
    ap.add_argument("--backend", default="auto", help="'auto' or 'cuda' (the only backend)")
    ap.add_argument("--device", type=int, default=0, help="CUDA device ordinal")
    ap.add_argument("--batch-size", type=int, default=1, help="sequences decoded in parallel")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="bfloat16 (serving kernels) or float32 (true 32-bit path)")
    ap.add_argument("--emit-stage-timings", action="store_true", help="print prefill/decode timings")
    ap.add_argument("--emit-generated-json", action="store_true",
                    help="print [generated_json] with the generated ids (and text, with a tokenizer)")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at stop tokens")
    return ap


def _tokenizer(model_dir):
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
    if args.backend not in ("auto", "cuda"):
        print(f"backend {args.backend!r} is not available: this build is CUDA sm_100a only", file=sys.stderr)
        return 2
    from .api import load
    from .config import load_config
    cfg = load_config(args.model_dir)
    if args.model and args.model.lower().replace("_", "-") not in ("llama", "llama3.1-8b", "llama3.2-3b",
                                                                     "llama3.2-1b", cfg.model_type):
        print(f"[warn] --model {args.model} is not a name this build knows; the folder's "
              f"architecture {cfg.architectures[0]} decides", file=sys.stderr)
    tok = _tokenizer(args.model_dir)
    prompts = [[int(t) for t in p.replace(" ", ",").split(",") if t] for p in args.prompt_ids]
    if args.prompt:
        if tok is None:
            print("--prompt needs tokenizer.json in the model folder and the tokenizers package; "
                  "use --prompt-ids", file=sys.stderr)
            return 2
        prompts.append(tok.encode(args.prompt, add_special_tokens=not args.prompt_no_special_tokens).ids)
    if not prompts:
        print("give --prompt-ids 1,2,3 (repeatable) or --prompt TEXT", file=sys.stderr)
        return 2
    longest = max(len(p) for p in prompts)
    context = args.context_size or (longest + args.max_new_tokens)
    batch = max(args.batch_size, 1)
    t0 = time.time()
    engine = load(args.model_dir, dtype=args.dtype, device=args.device, context_size=context,
                  batch_size=min(batch, len(prompts)))
    print(f"[weights] loaded in {(time.time() - t0) * 1e3:.0f}ms", file=sys.stderr)
    import torch
    first_done = []

    def on_step(live, tokens):
        if not first_done:
            torch.cuda.synchronize()
            first_done.append(time.time())
    t1 = time.time()
    from .sampling import SamplingParams
    results = engine.generator.generate(
        prompts, args.max_new_tokens,
        SamplingParams(args.temperature, args.top_k, args.top_p, args.sampling_seed),
        ignore_eos=args.ignore_eos, batch_size=batch, on_step=on_step)
    torch.cuda.synchronize()
    t2 = time.time()
    prefill_ms = ((first_done[0] if first_done else t2) - t1) * 1e3
    decode_ms = (t2 - (first_done[0] if first_done else t2)) * 1e3
    n_prompt = sum(len(p) for p in prompts[:batch])
    print(f"[prefill] {n_prompt} tokens in {prefill_ms:.0f}ms", file=sys.stderr)
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
    steps = max(engine.generator.steps_run - 1, 1)
    print(f"[result] prompt_tokens={sum(len(p) for p in prompts)} generated_tokens={n_gen} "
          f"decode_ms={decode_ms:.0f} ms_per_step={decode_ms / steps:.1f}", file=sys.stderr)
    if args.emit_stage_timings:
        print(f"[stage] prefill_ms={prefill_ms:.1f} decode_ms={decode_ms:.1f} steps={steps}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
