"""Norms.  ``rmsnorm``: y = x * rsqrt(mean(x^2) + eps) * w, statistics in float32,
one rounding at the end (kernels/full_attention_cuda.cuh:2826-2873; the weight is
used as ``w``, not ``1 + w``: crates/runner/src/llama31_engine.rs:89)."""
from __future__ import annotations

import torch

from .registry import BuildContext, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """params: ``size``, ``eps``; weights: ``weight`` [size].

    Interface of a norm: ``__call__(ctx, x, rows=None) -> tensor`` where ``x`` is the
    float32 residual stream ``[T, size]`` and the result has the activation dtype;
    ``rows`` (int32) picks rows of ``x`` instead of taking all.
    """

    fusable_rms = True     # kernels may apply this norm (weight, eps) inside a matrix product

    def __init__(self, params, weights, build: BuildContext):
        self.size, self.eps = int(params["size"]), float(params["eps"])
        w = build.weights.stored(weights["weight"])
        # 32-bit weights stay 32-bit; in the float32 path everything is 32-bit
        self.weight = w.float() if build.dtype == torch.float32 else w
        if tuple(self.weight.shape) != (self.size,):
            raise ValueError(f"rmsnorm weight has shape {tuple(self.weight.shape)}, expected ({self.size},)")
        self.dtype = build.dtype

    def __call__(self, ctx, x, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.dtype, device=x.device)
        ctx.kernels.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
