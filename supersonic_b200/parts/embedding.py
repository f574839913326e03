"""Token embedding: h[t] = E[id_t], widened into the float32 residual stream
(kernels/full_attention_cuda.cuh:2012-2034)."""
from __future__ import annotations

import torch

from .registry import BuildContext, register_embedding


@register_embedding("embedding")
class Embedding:
    """params: ``vocab_size``, ``hidden_size``; weights: ``weight`` [vocab, hidden]."""

    def __init__(self, params, weights, build: BuildContext):
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.table = build.weights.as_dtype(weights["weight"], build.dtype, share=True)
        if tuple(self.table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"{weights['weight']} has shape {tuple(self.table.shape)}, "
                             f"expected {(self.vocab, self.hidden)}")

    def __call__(self, ctx, token_ids):
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        ctx.kernels.embed(token_ids, self.table, out)
        return out
