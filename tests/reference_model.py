"""A whole LlamaForCausalLM prompt pass made of DeanoC/SuperSonic's own CUDA kernels.

The reference's model code is Rust and cannot be built here, but every arithmetic step of its
prompt pass is one of its CUDA kernels with a C launcher (``baseline/reference_kernels.py``
compiles them unmodified).  This module calls those kernels in the order and with the
roundings of the reference's prompt engine (crates/runner/src/prefill_engine.rs:1116-1222 for a
layer, :1954-2333 for attention, :3226-3366 for the feed-forward, :515-640 for the head): every
value between two kernels is bfloat16, rotary tables are rounded to bfloat16
(crates/runner/src/llama31_engine.rs:147-157), attention leaves float32 that is cast to
bfloat16.  Only data movement (row gather of the embedding, transposes between ``[T, H, D]`` and
``[H, T, D]``) is done with torch indexing; no arithmetic is.

It exists to pin ``plain_llama`` on the reference's own outputs and shares nothing with
``supersonic_b200``.
"""
import math

import numpy as np
import torch

import plain_llama as pl
from baseline import reference_kernels as rk


def _bf16(a, device):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device).to(torch.bfloat16).contiguous()


def forward(cfg, w, tokens, device="cuda:0"):
    """float32 logits [T, vocab] of one whole sequence, every operation a reference kernel."""
    T = len(tokens)
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nq
    hd = pl.head_dim_of(cfg)
    eps = cfg["rms_norm_eps"]
    cos64, sin64 = pl.rope_tables(cfg, T)
    cos, sin = _bf16(cos64, device), _bf16(sin64, device)
    W = {n: _bf16(a, device) for n, a in w.items()}
    ids = torch.tensor(list(tokens), dtype=torch.long, device=device)
    h = W["model.embed_tokens.weight"][ids].contiguous()
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}"
        x = rk.rms_norm(h, W[f"{p}.input_layernorm.weight"], eps)
        q = rk.matmul_rhs_transposed(x, W[f"{p}.self_attn.q_proj.weight"]).view(T, nq, hd)
        k = rk.matmul_rhs_transposed(x, W[f"{p}.self_attn.k_proj.weight"]).view(T, nkv, hd)
        v = rk.matmul_rhs_transposed(x, W[f"{p}.self_attn.v_proj.weight"]).view(T, nkv, hd)
        rk.apply_rope_prefill(q, cos, sin)
        rk.apply_rope_prefill(k, cos, sin)
        a = rk.attention_prefill(q.permute(1, 0, 2).contiguous()[None], k.permute(1, 0, 2).contiguous()[None],
                                 v.permute(1, 0, 2).contiguous()[None], 1.0 / math.sqrt(hd))
        a = a[0].to(torch.bfloat16).permute(1, 0, 2).reshape(T, nq * hd).contiguous()
        h = rk.element_add(h, rk.matmul_rhs_transposed(a, W[f"{p}.self_attn.o_proj.weight"]))
        x = rk.rms_norm(h, W[f"{p}.post_attention_layernorm.weight"], eps)
        z = rk.swiglu_mul(rk.matmul_rhs_transposed(x, W[f"{p}.mlp.gate_proj.weight"]),
                          rk.matmul_rhs_transposed(x, W[f"{p}.mlp.up_proj.weight"]))
        h = rk.element_add(h, rk.matmul_rhs_transposed(z, W[f"{p}.mlp.down_proj.weight"]))
    x = rk.rms_norm(h, W["model.norm.weight"], eps)
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return rk.matmul_rhs_transposed(x, head).float().cpu().numpy()
