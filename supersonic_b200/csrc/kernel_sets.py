"""Kernel sets: the operations parts call, bound to one family of kernels.

``PlainKernels`` runs every operation with the plain kernels (float32 arithmetic,
fixed summation order): it is the whole float32 path and also works with bfloat16
storage.  Faster sets derive from it and replace one operation at a time, each
checked against the plain one.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


class NormedInput:
    """The input of a mixer or feed-forward: ``norm(residual)``, not yet computed.

    ``tensor()`` runs the norm kernel (once) and gives the activations; a kernel set that
    can apply the norm inside its matrix product reads ``residual``, ``weight`` and
    ``eps`` instead and never materialises them."""

    def __init__(self, ctx, residual, norm):
        self.ctx, self.residual, self.norm = ctx, residual, norm
        self._tensor = None

    @property
    def fusable(self) -> bool:
        return getattr(self.norm, "fusable_rms", False)

    @property
    def weight(self):
        return self.norm.weight

    @property
    def eps(self) -> float:
        return self.norm.eps

    @property
    def n_rows(self) -> int:
        return self.residual.shape[0]

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.norm(self.ctx, self.residual)
        return self._tensor


def as_tensor(x) -> torch.Tensor:
    return x.tensor() if isinstance(x, NormedInput) else x


class PlainKernels:
    name = "plain"
    capturable = False      # the float32 path launches every step eagerly: each launch's status is looked at

    def embed(self, ids, table, out):
        ops.embed(ids, table, out)

    def rmsnorm(self, x, weight, eps, out, rows=None):
        ops.rmsnorm(x, weight, eps, out, rows)

    def linear(self, x, weight, out, accumulate=False):
        """out (+)= x @ weight^T; ``x`` may be a :class:`NormedInput`."""
        ops.gemm_nt_plain(as_tensor(x), weight, out, accumulate)

    def pack_gate_up(self, gate, up):
        """Gate and up weights as one matrix, in the layout ``gate_up_swiglu`` wants."""
        return torch.cat([gate, up], dim=0).contiguous(), "halves"

    def gate_up_swiglu(self, x, w_gate_up, layout, out):
        """out = silu(x @ gate^T) * (x @ up^T)."""
        x = as_tensor(x)
        gate_up = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
        self.linear(x, w_gate_up, gate_up)
        ops.swiglu(gate_up, out, interleaved=(layout == "interleaved"))

    def project_rope_append(self, x, w_qkv, qkv, position, kv, batch, n_q, n_kv, head_dim, page_shift) -> bool:
        """The q/k/v projection with position encoding and cache append in one kernel: rotated q
        into ``qkv``'s first columns, k and v into the cache.  False: not taken, nothing was done."""
        return False

    def rope_append(self, qkv, cos, sin, batch, page_table, k_cache, v_cache, n_q, n_kv, head_dim,
                    rotary_dim, page_shift, write_cache=True):
        ops.rope_append(qkv, cos, sin, batch.pos, batch.slot_of_token, page_table, k_cache, v_cache,
                        n_q, n_kv, head_dim, rotary_dim, page_shift, write_cache)

    def rope_attention(self, qkv, position, kv, batch, out, n_q, n_kv, head_dim, page_shift, window,
                       scale) -> bool:
        """Position encoding, cache append and attention in one launch, if this set can do it
        for this case; False means the caller runs the two steps separately."""
        return False

    def attention(self, q, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim, page_shift,
                  window: Optional[int], scale: float):
        ops.attention_plain(q, k_cache, v_cache, batch.pos, batch.slot_of_token, page_table, out,
                            n_q, n_kv, head_dim, page_shift, window, scale)

    def swiglu(self, gate_up, out):
        ops.swiglu(gate_up, out)

    def add_into(self, out, x):
        ops.add_into(out, x)

    def argmax(self, logits, out):
        ops.argmax(logits, out)

    def target_nll(self, logits, targets, out):
        ops.target_nll(logits, targets, out)

    def sample(self, logits, temperature, top_k, top_p, slots, rng_state, out, drawn_u=None):
        ops.sample(logits, temperature, top_k, top_p, slots, rng_state, out, drawn_u)


def kernel_set_for(dtype: torch.dtype, prefer: Optional[str] = None, deterministic: bool = False):
    """float32 always runs the plain set (which has no atomics on data); bfloat16 runs the fast set
    unless ``prefer='plain'``, with or without float atomics in its split projections."""
    if dtype == torch.float32 or prefer == "plain":
        return PlainKernels()
    from .fast_sets import FastKernels
    return FastKernels(deterministic=deterministic)
