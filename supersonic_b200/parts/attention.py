"""The attention mixer: grouped-query softmax attention over a sequence's cached keys.

q = x Wq^T, k = x Wk^T, v = x Wv^T (no bias); position encoding on q and k; k and v
appended to the cache at each token's position; for query head g and kv head
g // (n_q / n_kv): s_j = (q . k_j) * scale for the visible keys j, softmax in
float32 with the maximum subtracted, o = sum_j p_j v_j; out = o Wo^T added to the
residual (crates/runner/src/prefill_engine.rs:1912-2336;
crates/runner/src/decode_engine.rs:4303-4799, 8546-8774;
kernels/full_attention_cuda.cuh:360-576).  The three projections run as one
matrix product over row-concatenated weights.
"""
from __future__ import annotations

import torch

from ..cache import PAGE_SHIFT, KvNeed
from .registry import BuildContext, register_mixer


@register_mixer("attention")
class Attention:
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``,
    ``window`` (None = all earlier keys); weights: ``q``, ``k``, ``v``, ``o``.

    Interface of a mixer:
      ``cache_need()`` -> KvNeed | StateNeed | None
      ``forward(ctx, x, residual, cache_id, writes_cache, position)``: reads the normed
      activations ``x`` [T, hidden] and adds its output into ``residual`` (float32).
    """

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden = int(params["hidden_size"])
        self.n_q, self.n_kv = int(params["num_heads"]), int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = params.get("window")
        if self.n_q % self.n_kv:
            raise ValueError(f"{self.n_q} query heads do not split over {self.n_kv} kv heads")
        if self.head_dim % 16 or self.head_dim > 512:
            raise ValueError(f"head_dim {self.head_dim} is not supported: multiples of 16 up to 512")
        w = build.weights
        q, k, v = (w.as_dtype(weights[r], build.dtype) for r in ("q", "k", "v"))
        want = {"q": (self.n_q * self.head_dim, self.hidden), "k": (self.n_kv * self.head_dim, self.hidden),
                "v": (self.n_kv * self.head_dim, self.hidden), "o": (self.hidden, self.n_q * self.head_dim)}
        self.w_o = w.as_dtype(weights["o"], build.dtype)
        for r, t in (("q", q), ("k", k), ("v", v), ("o", self.w_o)):
            if tuple(t.shape) != want[r]:
                raise ValueError(f"{weights[r]} has shape {tuple(t.shape)}, expected {want[r]}")
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.n_q * self.head_dim]     # for a stop that only reads a cache
        self.dtype = build.dtype

    def cache_need(self):
        return KvNeed(self.n_kv, self.head_dim, self.window)

    @staticmethod
    def cache_need_from(params):
        """What ``cache_need()`` will say, from the parameters alone (asked before anything is built)."""
        return KvNeed(int(params["num_kv_heads"]), int(params["head_dim"]), params.get("window"))

    @staticmethod
    def activation_elements(params) -> int:
        """Elements per token this part holds while it runs: [q | k | v] and the attention output."""
        return (2 * int(params["num_heads"]) + 2 * int(params["num_kv_heads"])) * int(params["head_dim"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        T = ctx.batch.n_tokens
        kv = ctx.cache.kv(cache_id)
        width = (self.n_q + (2 * self.n_kv if writes_cache else 0)) * self.head_dim
        qkv = torch.empty((T, width), dtype=self.dtype, device=residual.device)
        attn = torch.empty((T, self.n_q * self.head_dim), dtype=self.dtype, device=residual.device)
        if writes_cache and ctx.kernels.project_rope_append(x, self.w_qkv, qkv, position, kv, ctx.batch, self.n_q,
                                                           self.n_kv, self.head_dim, PAGE_SHIFT):
            k_cache, v_cache, table, _ = kv          # q is rotated, k and v are in the cache
            ctx.kernels.attention(qkv, k_cache, v_cache, ctx.batch, table, attn, self.n_q, self.n_kv,
                                  self.head_dim, PAGE_SHIFT, self.window, self.scale)
            ctx.kernels.linear(attn, self.w_o, residual, accumulate=True)
            return
        ctx.kernels.linear(x, self.w_qkv if writes_cache else self.w_q, qkv)
        if not (writes_cache and ctx.kernels.rope_attention(qkv, position, kv, ctx.batch, attn, self.n_q,
                                                           self.n_kv, self.head_dim, PAGE_SHIFT,
                                                           self.window, self.scale)):
            position.encode_and_append(ctx, qkv, kv, self.n_q, self.n_kv, writes_cache)
            k_cache, v_cache, table, _ = kv
            ctx.kernels.attention(qkv, k_cache, v_cache, ctx.batch, table, attn, self.n_q, self.n_kv,
                                  self.head_dim, PAGE_SHIFT, self.window, self.scale)
        ctx.kernels.linear(attn, self.w_o, residual, accumulate=True)
