"""Builds traces for bin/trace_run, runs it as a user would (a subprocess fed through
standard input) and collects the logits it writes by (request, position)."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def rounded(n):
    return -(-n // 64) * 64


class Trace:
    def __init__(self):
        self.steps = []          # JSON records
        self.index = []          # per step: list of (request, position) in output order
        self.live_tokens = {}
        self.peak_tokens = 0

    def add(self, entries, end=()):
        """entries: list of (request id, tokens, first position, wanted places)."""
        rec = {"step": len(self.steps), "entries": [], "end": list(end)}
        idx = []
        for rid, tokens, first, want in entries:
            rec["entries"].append({"id": rid, "tokens": list(tokens), "want": list(want)})
            idx.extend((rid, first + w) for w in want)
            self.live_tokens[rid] = first + len(tokens)
        self.peak_tokens = max(self.peak_tokens, sum(rounded(n) for n in self.live_tokens.values()))
        for rid in end:
            del self.live_tokens[rid]
        self.steps.append(rec)
        self.index.append(idx)


def whole(trace, requests, tag="w"):
    """Each request alone, all its tokens in one step."""
    for rid, toks in requests.items():
        trace.add([(f"{tag}{rid}", toks, 0, range(len(toks)))], end=[f"{tag}{rid}"])


def tail_one_by_one(trace, requests, tail=32, tag="t"):
    """All but the last ``tail`` tokens in one step, then one token a step."""
    for rid, toks in requests.items():
        n0 = max(len(toks) - tail, 1)
        name = f"{tag}{rid}"
        trace.add([(name, toks[:n0], 0, range(n0))])
        for p in range(n0, len(toks)):
            trace.add([(name, [toks[p]], p, [0])], end=[name] if p == len(toks) - 1 else [])
        if n0 == len(toks):
            trace.add([], end=[name])


def batches(trace, requests, groups, prompt_of, tag="b"):
    """Batches that start together: each request's prompt in one step, then one token each per
    step; shorter requests end earlier; the next batch starts after the last request ended."""
    for group in groups:
        names = {rid: f"{tag}{rid}" for rid in group}
        done = {rid: prompt_of(rid, len(requests[rid])) for rid in group}
        first = [(names[r], requests[r][:done[r]], 0, range(done[r])) for r in group]
        trace.add(first, end=[names[r] for r in group if done[r] == len(requests[r])])
        live = [r for r in group if done[r] < len(requests[r])]
        while live:
            entries = [(names[r], [requests[r][done[r]]], done[r], [0]) for r in live]
            for r in live:
                done[r] += 1
            ended = [r for r in live if done[r] == len(requests[r])]
            trace.add(entries, end=[names[r] for r in ended])
            live = [r for r in live if r not in ended]


def run_trace(model_dir, dtype, trace, out_dir, max_tokens=None, vocab=None, env=None, timeout=600):
    """Runs bin/trace_run over the trace; returns {(request, position): logits row}."""
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens or trace.peak_tokens)]
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run exited {proc.returncode}\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(trace.steps))], proc.stdout[-2000:]
    out = {}
    for step, idx in enumerate(trace.index):
        path = os.path.join(out_dir, f"{step}.f32")
        if not idx:
            assert not os.path.exists(path)
            continue
        data = np.fromfile(path, dtype="<f4").reshape(len(idx), -1)
        if vocab is not None:
            assert data.shape[1] == vocab
        for key, row in zip(idx, data):
            assert key not in out, f"{key} written twice"
            out[key] = row
    return out
