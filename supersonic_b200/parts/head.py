"""Output head: logits = norm(h_row) W^T for the wanted rows only, float32 out
(crates/runner/src/prefill_engine.rs:515-640).  A tied head names the embedding's
tensor and shares its buffer (crates/runner/src/llama31_engine.rs:184-192)."""
from __future__ import annotations

import torch

from .registry import BuildContext, register_head


@register_head("linear_head")
class LinearHead:
    """params: ``vocab_size``, ``hidden_size``; weights: ``weight`` [vocab, hidden]."""

    def __init__(self, params, weights, build: BuildContext):
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.weight = build.weights.as_dtype(weights["weight"], build.dtype, share=True)
        if tuple(self.weight.shape) != (self.vocab, self.hidden):
            raise ValueError(f"{weights['weight']} has shape {tuple(self.weight.shape)}, "
                             f"expected {(self.vocab, self.hidden)}")

    def __call__(self, ctx, normed_rows):
        logits = torch.empty((normed_rows.shape[0], self.vocab), dtype=torch.float32,
                             device=normed_rows.device)
        ctx.kernels.linear(normed_rows, self.weight, logits)
        return logits
