"""Plain, slow implementation of the LlamaForCausalLM forward pass in NumPy float64.

Each function below cites the file and lines of DeanoC/SuperSonic whose arithmetic it restates.
The reference's model code is Rust and cannot be built without a Rust toolchain, but its CUDA
kernels can: ``baseline/reference_kernels.py`` compiles them unmodified, and
``tests/test_reference_ops_gpu.py`` pins each function here (norm, rotary pairing, SwiGLU,
projections, attention over a prompt and over a cache, the greedy tie rule, and a whole tiny
model chained as the reference chains it) on their outputs; ``tests/golden/
reference_kernels_logits.npz`` keeps such outputs for machines without a GPU.  What no kernel
computes (the llama3 frequency formula, which the reference evaluates in Rust:
crates/runner/src/llama31_engine.rs:115-145) rests on the formula alone.  Whole sequences, no
cache, one function per part; it reads the model folder with its own few lines and shares no
code with ``supersonic_b200``.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ---- model folder ---------------------------------------------------------------------
def read_model_folder(model_dir):
    """config.json as a dict and every tensor of model.safetensors as float64."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        weights[name] = arr.reshape(info["shape"])
    return cfg, weights


def head_dim_of(cfg):
    # default hidden/heads: crates/runner/src/llama31_engine.rs:72-76
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


# ---- parts ----------------------------------------------------------------------------
def rope_inv_freq(cfg):
    """llama3-scaled inverse frequencies (llama31_engine.rs:115-145)."""
    hd = head_dim_of(cfg)
    theta = cfg.get("rope_theta", 10000.0)
    sc = cfg.get("rope_scaling")
    out = []
    for i in range(hd // 2):
        base_inv = 1.0 / theta ** (2.0 * i / hd)
        if sc and sc.get("rope_type", "llama3") == "llama3":
            old = float(sc["original_max_position_embeddings"])
            low_wavelen = old / sc["low_freq_factor"]
            high_wavelen = old / sc["high_freq_factor"]
            wavelen = 2.0 * math.pi / base_inv
            if wavelen > low_wavelen:
                f = base_inv / sc["factor"]
            elif wavelen < high_wavelen:
                f = base_inv
            else:
                smooth = (old / wavelen - sc["low_freq_factor"]) / (
                    sc["high_freq_factor"] - sc["low_freq_factor"])
                f = (1.0 - smooth) * base_inv / sc["factor"] + smooth * base_inv
        else:
            f = base_inv
        out.append(f)
    return np.array(out, dtype=np.float64)


def rope_tables(cfg, n_positions):
    """cos/sin [n_positions, hd/2] of angle = pos * inv_freq (llama31_engine.rs:147-157;
    the reference then rounds the tables to bfloat16, which this does not)."""
    ang = np.arange(n_positions, dtype=np.float64)[:, None] * rope_inv_freq(cfg)[None, :]
    return np.cos(ang), np.sin(ang)


def apply_rope(x, cos, sin):
    """x [T, heads, hd]; half-split pairs (i, i+hd/2): kernels/prefill_helpers_cuda.cuh:80-111."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1)


def rms_norm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w (kernels/full_attention_cuda.cuh:2826-2873,
    weight used as w, not 1+w: llama31_engine.rs:89)."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def embedding(tokens, table):
    """h[t] = E[id_t] (kernels/full_attention_cuda.cuh:2012-2034)."""
    return table[np.asarray(tokens, dtype=np.int64)]


def attention_scores(q, k, v, scale, window=None):
    """Causal GQA attention over whole sequences, q [T,nq,hd], k/v [T,nkv,hd].
    Query head g reads kv head g // (nq/nkv); keys j <= t (and j > t - window);
    max-subtracted softmax; (kernels/full_attention_cuda.cuh:360-474;
    crates/kernel-ffi/src/metal_host.rs:1330-1404)."""
    T, nq, hd = q.shape
    group = nq // k.shape[1]
    out = np.zeros_like(q)
    for g in range(nq):
        kk, vv = k[:, g // group], v[:, g // group]
        s = (q[:, g] @ kk.T) * scale
        j = np.arange(T)
        mask = j[None, :] > j[:, None]
        if window is not None:
            mask |= j[None, :] <= j[:, None] - window
        s = np.where(mask, -np.inf, s)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, g] = (p @ vv) / p.sum(axis=-1, keepdims=True)
    return out


def attention_mixer(x, w, prefix, cfg, cos, sin, window=None):
    """q/k/v projections, rotary on q and k, attention, output projection
    (crates/runner/src/prefill_engine.rs:1954-2324; scale 1/sqrt(hd) at :2200)."""
    T = x.shape[0]
    nq, nkv, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg[
        "num_attention_heads"], head_dim_of(cfg)
    q = (x @ w[f"{prefix}.self_attn.q_proj.weight"].T).reshape(T, nq, hd)
    k = (x @ w[f"{prefix}.self_attn.k_proj.weight"].T).reshape(T, nkv, hd)
    v = (x @ w[f"{prefix}.self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
    q, k = apply_rope(q, cos[:T], sin[:T]), apply_rope(k, cos[:T], sin[:T])
    a = attention_scores(q, k, v, 1.0 / math.sqrt(hd), window).reshape(T, nq * hd)
    return a @ w[f"{prefix}.self_attn.o_proj.weight"].T


def swiglu_ffn(x, w, prefix):
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g))
    (crates/runner/src/prefill_engine.rs:3226-3366; kernels/full_attention_cuda.cuh:1995-2010)."""
    g = x @ w[f"{prefix}.mlp.gate_proj.weight"].T
    u = x @ w[f"{prefix}.mlp.up_proj.weight"].T
    return (g / (1.0 + np.exp(-g)) * u) @ w[f"{prefix}.mlp.down_proj.weight"].T


def block(h, w, n, cfg, cos, sin):
    """Pre-norm residual block (prefill_engine.rs:1116-1222)."""
    p = f"model.layers.{n}"
    eps = cfg["rms_norm_eps"]
    h = h + attention_mixer(rms_norm(h, w[f"{p}.input_layernorm.weight"], eps), w, p, cfg, cos, sin)
    h = h + swiglu_ffn(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, p)
    return h


def output_head(h, w, cfg):
    """Final norm and logits; a tied head reuses the embedding
    (prefill_engine.rs:515-640; llama31_engine.rs:184-192)."""
    n = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return n @ head.T


def forward(cfg, w, tokens):
    """Logits [T, vocab] (float64) at every position of one whole sequence."""
    cos, sin = rope_tables(cfg, len(tokens))
    h = embedding(tokens, w["model.embed_tokens.weight"])
    for n in range(cfg["num_hidden_layers"]):
        h = block(h, w, n, cfg, cos, sin)
    return output_head(h, w, cfg)


# ---- sampling and generation ----------------------------------------------------------
def greedy_token(logits):
    """argmax with strict '>', so the lowest index wins ties
    (crates/runner/src/decode_engine.rs:11162-11172)."""
    best, best_v = 0, -math.inf
    for i, v in enumerate(logits):
        if v > best_v:
            best, best_v = i, v
    return best


def sampling_distribution(logits, temperature, top_k=0, top_p=1.0):
    """Probabilities after temperature, top-k and top-p
    (crates/runner/src/qwen36_moe_decode.rs:1115-1185): scale by 1/T, keep the k
    largest, softmax over them, keep the smallest prefix (largest first) whose
    mass reaches top_p, renormalise.  Ties at a cut are all kept."""
    x = np.asarray(logits, dtype=np.float64) / temperature
    keep = np.ones(x.shape, dtype=bool)
    if top_k and top_k < x.size:
        kth = np.sort(x)[::-1][top_k - 1]
        keep &= x >= kth
    p = np.where(keep, np.exp(x - x[keep].max()), 0.0)
    p /= p.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cum = np.cumsum(p[order])
        n = int(np.searchsorted(cum, top_p, side="left")) + 1
        cut = p[order[min(n, x.size) - 1]]
        p = np.where(p >= cut, p, 0.0)
        p /= p.sum()
    return p


def greedy_generate(cfg, w, prompt, max_new_tokens, stop_ids=()):
    """Whole-sequence re-run per token; the stop token is kept, as in the
    reference's loop (llama31_engine.rs:1185-1197, 1549-1550)."""
    tokens, out = list(prompt), []
    while len(out) < max_new_tokens:
        nxt = greedy_token(forward(cfg, w, tokens)[-1])
        out.append(nxt)
        tokens.append(nxt)
        if nxt in stop_ids:
            break
    return out
