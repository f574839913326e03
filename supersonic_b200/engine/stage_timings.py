"""Where a step's device time goes, by stage, behind a switch.

The reference brackets every stage of a decode step with host timers and a forced device
synchronise when ``--emit-stage-timings`` is given, sums them in ``DecodeStageTimings`` and
prints one ``[stage]`` line (crates/runner/src/decode_engine.rs:1101-1232, 10157-10162;
crates/runner/src/llama31_engine.rs:432-463).  Here :class:`TimedKernels` stands in front of the
model's kernel set for the steps that are timed: every operation a part asks for is bracketed by
two CUDA events on the launching stream, and filed under a stage named after the reference's:

    embed, rms_norm, full_attn_proj (q/k/v and output projections), full_attn_core (position
    encoding, cache append, attention), mlp, lm_head, sampling

The stage comes from which part is running (``ctx.stage``, set by the model and by the block
arrangement) and from the operation.  Timed steps run uncaptured and their kernels do not overlap
each other across an event, so the sum is larger than an untimed step: the shares are what
the figures are for.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

STAGES = ("embed", "rms_norm", "full_attn_proj", "full_attn_core", "mlp", "lm_head", "sampling", "other")
_CORE_OPS = {"attention", "rope_attention", "rope_append"}


def stage_of(part: str, op: str) -> str:
    if op == "rmsnorm":
        return "rms_norm"
    if op == "embed":
        return "embed"
    if op in ("argmax", "sample"):
        return "sampling"
    if part == "mixer":
        return "full_attn_core" if op in _CORE_OPS else "full_attn_proj"
    if part == "feed_forward":
        return "mlp"
    if part == "head":
        return "lm_head"
    return "other"


class TimedKernels:
    """A kernel set whose operations are bracketed by CUDA events.  ``ctx`` is the running step's
    context (its ``stage`` names the part); an operation that runs inside another (a norm computed
    on demand inside a projection) is taken out of its parent's time."""

    def __init__(self, inner):
        self._inner = inner
        self.ctx = None
        self._open: List[int] = []
        self._records: List[list] = []       # [stage, start event, end event, parent index]

    def __getattr__(self, name):
        attr = getattr(self._inner, name)
        if name.startswith("_") or not callable(attr) or name == "pack_gate_up":
            return attr

        def timed(*args, **kwargs):
            part = getattr(self.ctx, "stage", "") if self.ctx is not None else ""
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            me = len(self._records)
            self._records.append([stage_of(part, name), start, end, self._open[-1] if self._open else -1])
            self._open.append(me)
            start.record()
            try:
                return attr(*args, **kwargs)
            finally:
                end.record()
                self._open.pop()
        return timed

    def collect(self) -> Dict[str, float]:
        """Milliseconds per stage since the last call (waits for the device)."""
        torch.cuda.synchronize()
        ms = [r[1].elapsed_time(r[2]) for r in self._records]
        own = list(ms)
        for i, r in enumerate(self._records):
            if r[3] >= 0:
                own[r[3]] -= ms[i]
        out = {s: 0.0 for s in STAGES}
        for r, t in zip(self._records, own):
            out[r[0]] += max(t, 0.0)
        self._records.clear()
        return out


class StageTimings:
    """Sums over the timed steps of a run, and the ``[stage]`` line."""

    def __init__(self):
        self.ms = {s: 0.0 for s in STAGES}
        self.tokens = 0
        self.steps = 0

    def add(self, ms: Dict[str, float], tokens: int) -> None:
        for k, v in ms.items():
            self.ms[k] = self.ms.get(k, 0.0) + v
        self.tokens += tokens
        self.steps += 1

    @property
    def total_ms(self) -> float:
        return sum(self.ms.values())

    def line(self, label: Optional[str] = None) -> str:
        if not self.tokens:
            return "[stage] tokens=0"
        head = f"[stage] {label + ' ' if label else ''}tokens={self.tokens} steps={self.steps} " \
               f"total_ms={self.total_ms:.1f} per_tok_ms={self.total_ms / self.tokens:.3f}"
        full_attn = self.ms["full_attn_proj"] + self.ms["full_attn_core"]
        body = f" full_attn={full_attn:.1f}" + "".join(
            f" {s}={self.ms[s]:.1f}" for s in STAGES if s != "other" or self.ms[s] > 0)
        return head + body
