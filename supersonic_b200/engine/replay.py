"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  The program drives the same :class:`Model`, step function,
cache and kernels that generation uses; it has no forward pass of its own.  It is
the batch-capable descendant of the reference's validators: ``--gpu-validate``
re-runs the whole history for every decoded token
(crates/runner/src/prefill_engine.rs:1505-1530, llama31_engine.rs:1266-1302) and
``--teacher-forced`` feeds given tokens (llama31_engine.rs:481-707).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` bring each request's next tokens and the places among them whose logits
are wanted; ``end`` lists requests that are finished after the step (their slot and
pages are given back).  For a step with wanted places, ``<out>/<step>.f32`` holds the
logits ``[wanted, vocab]`` as little-endian float32 in the order of the entries and
of ``want``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

from .batch import StepEntry
from .model import Model


class Replayer:
    """Request ids to slots; one :meth:`run_step` per input line."""

    def __init__(self, model: Model, out_dir: str):
        self.model, self.out_dir = model, out_dir
        self.slot_of: Dict[str, int] = {}
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, record: dict) -> None:
        step = record["step"]
        entries = []
        for e in record.get("entries", []):
            rid = str(e["id"])
            if rid not in self.slot_of:
                self.slot_of[rid] = self.model.open_sequence()
            entries.append(StepEntry(self.slot_of[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = self.model.step(entries)
            if logits.shape[0]:
                data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                self.model.check_errors()
                tmp = os.path.join(self.out_dir, f".{step}.f32.tmp")
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(self.out_dir, f"{step}.f32"))
        for rid in record.get("end", []):
            rid = str(rid)
            if rid not in self.slot_of:
                raise ValueError(f"step {step}: request {rid!r} ends but never started")
            self.model.close_sequence(self.slot_of.pop(rid))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    model = Model.from_dir(args.model, dtype=args.dtype, device=f"cuda:{args.device}",
                           max_tokens=args.max_tokens)
    replayer = Replayer(model, args.out)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        replayer.run_step(record)
        sys.stdout.write(f"done {record['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
