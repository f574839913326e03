"""Feed-forwards.  ``swiglu``: down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g)),
added to the residual (crates/runner/src/prefill_engine.rs:3226-3366;
kernels/full_attention_cuda.cuh:1995-2010).  Gate and up run as one matrix product
over row-concatenated weights."""
from __future__ import annotations

import torch

from .registry import BuildContext, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    """params: ``hidden_size``, ``intermediate_size``; weights: ``gate``, ``up``, ``down``.

    Interface of a feed-forward: ``forward(ctx, x, residual)`` reads the normed
    activations ``x`` [T, hidden] and adds its output into ``residual`` (float32).
    """

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        w = build.weights
        gate, up = w.as_dtype(weights["gate"], build.dtype), w.as_dtype(weights["up"], build.dtype)
        self.w_down = w.as_dtype(weights["down"], build.dtype)
        for name, t, want in ((weights["gate"], gate, (self.inter, self.hidden)),
                              (weights["up"], up, (self.inter, self.hidden)),
                              (weights["down"], self.w_down, (self.hidden, self.inter))):
            if tuple(t.shape) != want:
                raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {want}")
        self.w_gate_up, self.layout = build.kernels.pack_gate_up(gate, up)
        self.dtype = build.dtype

    @staticmethod
    def activation_elements(params) -> int:
        """Elements per token this part holds while it runs: gate and up, and their product."""
        return 3 * int(params["intermediate_size"])

    def forward(self, ctx, x, residual):
        z = torch.empty((residual.shape[0], self.inter), dtype=self.dtype, device=residual.device)
        ctx.kernels.gate_up_swiglu(x, self.w_gate_up, self.layout, z)
        ctx.kernels.linear(z, self.w_down, residual, accumulate=True)
