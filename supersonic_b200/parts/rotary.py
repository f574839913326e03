"""Position encodings.  ``rotary``: tables of cos/sin(pos * f_i) with the llama3
frequency scaling, built in float64 and kept in float32
(crates/runner/src/llama31_engine.rs:115-168; the reference rounds its tables to
bfloat16, which this engine does not: angles and their functions stay 32-bit).
``none``: no position information is added (keys are stored as they are)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .registry import BuildContext, register_position_encoding


def scaled_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = theta^(-2i/d); llama3 scaling divides low frequencies by ``factor``, keeps
    high ones and blends in between (llama31_engine.rs:126-145).  float64."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (2.0 * i / rotary_dim))
    if not scaling:
        return inv
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    old = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv
    smooth = (old / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen > old / low, inv / factor,
                       torch.where(wavelen < old / high, inv, blended))


@register_position_encoding("rotary")
class Rotary:
    """params: ``head_dim``, ``rotary_dim``, ``theta``, ``max_positions``, ``scaling``.

    Interface of a position encoding: ``encode_and_append(ctx, qkv, kv, n_q, n_kv, write)``
    rotates the queries (and keys) of the packed ``qkv`` rows in place by each
    token's position and writes keys and values into the cache entry ``kv``.
    """

    def __init__(self, params, weights, build: BuildContext):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        n_pos = min(int(params["max_positions"]), int(build.max_positions))
        self.max_positions = n_pos
        inv = scaled_inverse_frequencies(self.rotary_dim, float(params["theta"]), params.get("scaling"))
        angle = torch.arange(n_pos, dtype=torch.float64, device=build.device)[:, None] \
            * inv.to(build.device)[None, :]
        self.cos = angle.cos().to(torch.float32).contiguous()
        self.sin = angle.sin().to(torch.float32).contiguous()

    def check_range(self, batch) -> None:
        if batch.max_total > self.max_positions:
            raise ValueError(f"a sequence reaches {batch.max_total} tokens, beyond the "
                             f"{self.max_positions} positions this model encodes")

    def rotary_tables(self):
        """(cos, sin, rotary_dim) for kernels that rotate inside another operation."""
        return self.cos, self.sin, self.rotary_dim

    def encode_and_append(self, ctx, qkv, kv, n_q, n_kv, write_cache=True):
        self.check_range(ctx.batch)
        k_cache, v_cache, table, group = kv
        from ..cache import PAGE_SHIFT
        ctx.kernels.rope_append(qkv, self.cos, self.sin, ctx.batch, table, k_cache, v_cache, n_q, n_kv,
                                self.head_dim, self.rotary_dim, PAGE_SHIFT, write_cache)


@register_position_encoding("none")
class NoPosition:
    def __init__(self, params, weights, build: BuildContext):
        self.head_dim = int(params["head_dim"])

    def encode_and_append(self, ctx, qkv, kv, n_q, n_kv, write_cache=True):
        k_cache, v_cache, table, group = kv
        from ..cache import PAGE_SHIFT
        ctx.kernels.rope_append(qkv, None, None, ctx.batch, table, k_cache, v_cache, n_q, n_kv,
                                self.head_dim, 0, PAGE_SHIFT, write_cache)
