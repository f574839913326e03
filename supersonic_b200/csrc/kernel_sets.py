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


class PlainKernels:
    name = "plain"

    def embed(self, ids, table, out):
        ops.embed(ids, table, out)

    def rmsnorm(self, x, weight, eps, out, rows=None):
        ops.rmsnorm(x, weight, eps, out, rows)

    def linear(self, x, weight, out, accumulate=False):
        """out (+)= x @ weight^T."""
        ops.gemm_nt_plain(x, weight, out, accumulate)

    def rope_append(self, qkv, cos, sin, batch, page_table, k_cache, v_cache, n_q, n_kv, head_dim,
                    rotary_dim, page_shift, write_cache=True):
        ops.rope_append(qkv, cos, sin, batch.pos, batch.slot_of_token, page_table, k_cache, v_cache,
                        n_q, n_kv, head_dim, rotary_dim, page_shift, write_cache)

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

    def sample(self, logits, temperature, top_k, top_p, slots, rng_state, out, drawn_u=None):
        ops.sample(logits, temperature, top_k, top_p, slots, rng_state, out, drawn_u)


def kernel_set_for(dtype: torch.dtype, prefer: Optional[str] = None):
    """float32 always runs the plain set; bfloat16 runs the fast set unless ``prefer='plain'``."""
    if dtype == torch.float32 or prefer == "plain":
        return PlainKernels()
    from .fast_sets import FastKernels
    return FastKernels()
