"""Teacher-forced scoring: feed given tokens, score each next token under the model.

The reference's ``--teacher-forced`` runs the prompt (scoring every position on the device) or,
in its legacy mode, one token as the prompt and then one decode step per token, and reports
total and mean negative log-likelihood, perplexity and bits per token
(crates/runner/src/llama31_engine.rs:465-707; kernels/prefill_helpers_bridge_cuda.cu:405-520).
Here a batch of sequences is scored through the same step function that generation uses;
nothing is sampled.  Logits of many positions are large (vocabulary x 4 bytes a row), so the
prompt is fed in pieces of at most ``rows_per_step`` scored positions per sequence, each piece
continuing from the cache the one before left.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import List, Sequence

import torch

from .batch import StepEntry


@dataclass
class Score:
    tokens: int = 0
    scored_tokens: int = 0
    total_nll: float = 0.0
    decode_steps: int = 0
    total_ms: float = 0.0

    @property
    def avg_nll(self) -> float:
        return self.total_nll / self.scored_tokens

    @property
    def perplexity(self) -> float:
        return math.exp(self.avg_nll)

    @property
    def bits_per_token(self) -> float:
        return self.avg_nll / math.log(2.0)

    def to_dict(self) -> dict:
        return {"prompt_tokens": self.tokens, "scored_tokens": self.scored_tokens, "decode_steps": self.decode_steps,
                "total_nll": self.total_nll, "avg_nll": self.avg_nll, "perplexity": self.perplexity,
                "bits_per_token": self.bits_per_token, "total_ms": self.total_ms,
                "ms_per_token": self.total_ms / max(self.scored_tokens, 1)}


def _nll(model, logits: torch.Tensor, targets: Sequence[int]) -> torch.Tensor:
    t = torch.tensor(list(targets), dtype=torch.int32).to(logits.device, non_blocking=True)
    out = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    model.kernels.target_nll(logits, t, out)
    return out


def teacher_forced(model, sequences: Sequence[Sequence[int]], decode_step: bool = False,
                   rows_per_step: int = 256) -> List[Score]:
    """Score ``sequences`` (each at least two tokens) as one batch that starts together.
    ``decode_step``: the first token is the prompt and every other token is fed in a decode step of
    its own (the reference's ``--teacher-forced-decode-step``); otherwise prompts run in pieces."""
    seqs = [list(s) for s in sequences]
    for i, s in enumerate(seqs):
        if len(s) < 2:
            raise ValueError(f"sequence {i}: teacher-forced scoring needs at least 2 tokens")
    t0 = time.perf_counter()
    scores = [Score(tokens=len(s)) for s in seqs]
    slots = [model.open_sequence() for _ in seqs]
    sums = [[] for _ in seqs]
    try:
        done = [0] * len(seqs)             # tokens fed so far
        first = True
        while True:
            entries, who = [], []
            for i, s in enumerate(seqs):
                left = len(s) - 1 - done[i]          # the last token is a target only
                if left <= 0:
                    continue
                n = 1 if decode_step else min(left, rows_per_step)
                entries.append(StepEntry(slots[i], s[done[i]:done[i] + n], range(n)))
                who.append((i, n))
            if not entries:
                break
            logits = model.step(entries)
            targets = [t for i, n in who for t in seqs[i][done[i] + 1:done[i] + n + 1]]
            nll = _nll(model, logits, targets)
            row = 0
            for i, n in who:
                sums[i].append(nll[row:row + n].double().sum())
                scores[i].scored_tokens += n
                if not first and n == 1:
                    scores[i].decode_steps += 1
                row += n
                done[i] += n
            first = False
        for i in range(len(seqs)):
            scores[i].total_nll = float(torch.stack(sums[i]).sum().item())
        model.check_errors()
    finally:
        for s in slots:
            model.close_sequence(s)
    ms = (time.perf_counter() - t0) * 1e3
    for sc in scores:
        sc.total_ms = ms
    return scores
