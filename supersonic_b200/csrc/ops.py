"""Python faces of the plain CUDA kernels: tensors in, a launch on the current stream out.

Every wrapper checks what the kernel assumes (device, dtype, contiguity, sizes)
and raises; a non-zero status from the library raises :class:`KernelError`.
There is no CPU path: without a CUDA device, or without the compiled library,
these functions fail.  One wrapper per op, like the reference's
``prefill_ffi`` (crates/kernel-ffi/src/prefill_ffi.rs:1104-3292) with its dtype
codes (crates/gpu-hal/src/scalar_type.rs:25-32).
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {2001: "unsupported dtype", 2002: "unsupported size", 2003: "unsupported configuration",
           2004: "a bounded wait ran out"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status:
        reason = _ERRORS.get(status) or f"CUDA error {status}"
        raise KernelError(f"{what}: {reason}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle (the raw query is several times cheaper than building a
    ``torch.cuda.Stream`` object, and this runs for every launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None, rows_contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dims, has shape {tuple(t.shape)}")
    if rows_contiguous and t.dim() >= 1 and t.numel() and t.stride(-1) != 1:
        raise KernelError(f"{name} must be contiguous in its last dim")
    if t.dim() > 2 and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_lib_cache = {}
LAUNCHES = 0          # kernels launched through this module (graph replays are counted by their owner)


def _fn(lib: str, name: str):
    key = (lib, name)
    if key not in _lib_cache:
        f = getattr(load_library(lib), name)
        f.restype = c_int
        _lib_cache[key] = f
    return _lib_cache[key]


# ---- plain ops -------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] into the float32 residual stream."""
    _need(ids, "ids", torch.int32, 1); _need(table, "table", None, 2); _need(out, "out", torch.float32, 2)
    if not (table.is_contiguous() and out.is_contiguous()):
        raise KernelError("embed: table and out must be contiguous")
    if out.shape[0] != ids.shape[0] or out.shape[1] != table.shape[1]:
        raise KernelError(f"embed: out {tuple(out.shape)} does not fit {ids.shape[0]} ids of width {table.shape[1]}")
    _check(_fn("plain_ops", "ssb_embed")(
        _ptr(ids), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(out), c_int(ids.shape[0]),
        c_int(table.shape[1]), c_int(table.shape[0]), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight, x float32."""
    _need(x, "x", torch.float32, 2); _need(weight, "weight", None, 1); _need(out, "out", None, 2)
    if not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("rmsnorm: x and out must be contiguous")
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] != n:
            raise KernelError("rmsnorm: one output row per gathered row")
    elif x.shape[0] != n:
        raise KernelError("rmsnorm: x and out differ in rows")
    if x.shape[1] != out.shape[1] or weight.shape[0] != x.shape[1]:
        raise KernelError("rmsnorm: widths differ")
    _check(_fn("plain_ops", "ssb_rmsnorm")(
        _ptr(x), _ptr(rows), _ptr(weight), c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(n), c_int(x.shape[1]), c_int(1 if pdl else 0), _stream()), "rmsnorm")


def gemm_nt_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[m, n] (+)= sum_k a[m, k] w[n, k]; float32 accumulation in k order."""
    _need(a, "a", None, 2); _need(w, "w", None, 2); _need(out, "out", None, 2)
    if a.dtype != w.dtype:
        raise KernelError(f"gemm: a is {a.dtype} but w is {w.dtype}")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("plain_ops", "ssb_gemm_nt_plain")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), c_int(dtype_code(a.dtype)), _ptr(out),
        c_int(out.stride(0)), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_int(1 if accumulate else 0), _stream()), "gemm_nt_plain")


def rope_append(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                pos: torch.Tensor, slot: torch.Tensor, page_table: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_q: int, n_kv: int,
                head_dim: int, rotary_dim: int, page_shift: int, write_cache: bool = True) -> None:
    """Rotate q (and k) of every token in place; write k and v into the paged cache entry."""
    _need(qkv, "qkv", None, 2); _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    T = qkv.shape[0]
    if qkv.shape[1] < (n_q + 2 * n_kv) * head_dim and write_cache:
        raise KernelError("rope_append: qkv rows are too narrow")
    if pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("rope_append: one position and one slot per token")
    table_positions = 0
    if cos is not None:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] != rotary_dim // 2 or not cos.is_contiguous() \
                or not sin.is_contiguous():
            raise KernelError("rope_append: cos/sin must be [positions, rotary_dim/2], contiguous")
        table_positions = cos.shape[0]
    if write_cache:
        for c in (k_cache, v_cache):
            _need(c, "cache", qkv.dtype)
            if not c.is_contiguous():
                raise KernelError("rope_append: cache entry must be contiguous")
    _check(_fn("plain_ops", "ssb_rope_append")(
        _ptr(qkv), c_int(qkv.stride(0)), c_int(dtype_code(qkv.dtype)), _ptr(cos), _ptr(sin),
        c_int(table_positions), _ptr(pos), _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]),
        _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim),
        c_int(rotary_dim), c_int(page_shift), c_int(1 if write_cache else 0), _stream()), "rope_append")


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                    slot: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                    head_dim: int, page_shift: int, window: Optional[int], scale: float) -> None:
    """Each token attends over keys [max(0, pos-window+1), pos] of its slot in the paged cache."""
    _need(q, "q", None, 2); _need(out, "out", q.dtype, 2)
    _need(k_cache, "k_cache", q.dtype); _need(v_cache, "v_cache", q.dtype)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    T = q.shape[0]
    if out.shape[0] != T or out.shape[1] < n_q * head_dim or q.shape[1] < n_q * head_dim:
        raise KernelError("attention: q/out shapes")
    if head_dim > 512 or n_q % n_kv:
        raise KernelError(f"attention_plain: head_dim {head_dim} (max 512), heads {n_q}/{n_kv} not supported")
    _check(_fn("plain_ops", "ssb_attention_plain")(
        _ptr(q), c_int(q.stride(0)), c_int(dtype_code(q.dtype)), _ptr(k_cache), _ptr(v_cache), _ptr(pos),
        _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)),
        c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(page_shift),
        c_int(int(window) if window else 0), c_float(scale), _stream()), "attention_plain")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[t, c] = silu(gate[t, c]) * up[t, c]; gate and up are the halves of a row of
    ``gate_up``, or (interleaved) alternate as [8 gate | 8 up] per 16 columns."""
    _need(gate_up, "gate_up", None, 2); _need(out, "out", gate_up.dtype, 2)
    T, inter = out.shape
    if gate_up.shape[0] != T or gate_up.shape[1] != 2 * inter:
        raise KernelError("swiglu: gate_up must be [T, 2*I] for out [T, I]")
    _check(_fn("plain_ops", "ssb_swiglu")(
        _ptr(gate_up), c_int(gate_up.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(T), c_int(inter), c_int(1 if interleaved else 0),
        _stream()), "swiglu")


def add_into(out: torch.Tensor, x: torch.Tensor) -> None:
    """out (float32) += x."""
    _need(out, "out", torch.float32); _need(x, "x")
    if not (out.is_contiguous() and x.is_contiguous()) or out.numel() != x.numel():
        raise KernelError("add_into: contiguous tensors of equal size")
    _check(_fn("plain_ops", "ssb_add_into")(
        _ptr(out), _ptr(x), c_int(dtype_code(x.dtype)), c_longlong(out.numel()), _stream()), "add_into")


# ---- sampling --------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax: one output per row")
    _check(_fn("sampling", "ssb_argmax")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(logits.shape[0]), c_int(logits.shape[1]),
        _ptr(out), _stream()), "argmax")


def target_nll(logits: torch.Tensor, targets: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = -log softmax(logits[r])[targets[r]] (float32; NaN for a target outside the vocabulary)."""
    _need(logits, "logits", torch.float32, 2); _need(targets, "targets", torch.int32, 1)
    _need(out, "out", torch.float32, 1)
    if targets.shape[0] != logits.shape[0] or out.shape[0] != logits.shape[0]:
        raise KernelError("target_nll: one target and one output per row")
    _check(_fn("sampling", "ssb_target_nll")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(logits.shape[0]), c_int(logits.shape[1]),
        _ptr(targets), _ptr(out), _stream()), "target_nll")


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
           slots: Optional[torch.Tensor], rng_state: torch.Tensor, out: torch.Tensor,
           drawn_u: Optional[torch.Tensor] = None) -> None:
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    _need(rng_state, "rng_state", torch.int64, 1)
    n = logits.shape[0]
    if slots is not None:
        _need(slots, "slots", torch.int32, 1)
        if slots.shape[0] != n:
            raise KernelError("sample: one slot per row")
    elif rng_state.shape[0] < n:
        raise KernelError("sample: one generator state per row")
    if drawn_u is not None:
        _need(drawn_u, "drawn_u", torch.float32, 1)
    if out.shape[0] != n:
        raise KernelError("sample: one output per row")
    _check(_fn("sampling", "ssb_sample")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(n), c_int(logits.shape[1]),
        c_float(temperature), c_int(int(top_k)), c_float(top_p), _ptr(slots), _ptr(rng_state), _ptr(out),
        _ptr(drawn_u), _stream()), "sample")


# ---- decode kernels --------------------------------------------------------------------
SG_STORE, SG_ACCUMULATE, SG_SWIGLU = 0, 1, 2


def skinny_gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the skinny GEMM takes these operands (else the plain kernels do)."""
    return (w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and x.shape[0] <= 64 and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def skinny_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = SG_STORE,
                pdl: bool = False) -> None:
    """out = x @ w^T for up to 64 rows on mma.sync (the decode projection for shapes the tcgen05
    kernels refuse).  ``pdl``: launch as a programmatic dependent of the kernel before it on the
    stream (its weights are prefetched while that kernel ends).  mode: store, add into float32
    ``out``, or SwiGLU over rows of ``w`` that come as [8 gate | 8 up] per 16 (``out`` is [rows, N/2])."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", None, 2)
    B, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if mode == SG_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (B, n_out):
        raise KernelError(f"skinny_gemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("decode_ops", "ssb_skinny_gemm")(
        _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(B), c_int(N), c_int(K), c_int(mode), c_int(1 if pdl else 0),
        _stream()), "skinny_gemm")


def attention_decode_scratch(n_seqs: int, n_q: int, n_kv: int, head_dim: int, n_splits: int):
    """(float32 elements of scratch, int32 counters) one launch needs; counters start at zero."""
    lib = load_library("decode_ops")
    lib.ssb_attention_decode_scratch_floats.restype = c_longlong
    return (int(lib.ssb_attention_decode_scratch_floats(c_int(n_seqs), c_int(n_q), c_int(head_dim),
                                                        c_int(n_splits))),
            int(lib.ssb_attention_decode_counters(c_int(n_seqs), c_int(n_q), c_int(n_kv))))


def _attention_decode_checks(q, k_cache, v_cache, pos, slot, page_table, out, n_q, n_kv, head_dim, cos, sin, what):
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    B = q.shape[0]
    if pos.shape[0] != B or slot.shape[0] != B or out.shape[0] != B:
        raise KernelError(f"{what}: one position, slot and output row per sequence")
    if cos is not None:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != head_dim or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError(f"{what}: cos/sin must be [positions, head_dim/2], contiguous")
        if head_dim not in (32, 64, 128, 256) or q.shape[1] < (n_q + 2 * n_kv) * head_dim:
            raise KernelError(f"{what}: fused rotation needs head_dim 32/64/128/256 and [q|k|v] rows")
    return B


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                     slot: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, page_shift: int, window: Optional[int], scale: float, n_splits: int,
                     scratch: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                     pdl: bool = False, cos: Optional[torch.Tensor] = None,
                     sin: Optional[torch.Tensor] = None) -> None:
    """One query token per sequence (row) over its cached keys, the keys split ``n_splits`` ways, on
    CUDA cores (any head size up to 256).  With ``cos``/``sin`` ([positions, head_dim/2] float32) the
    rows of ``q`` are the raw fused projection [q | k | v]: queries and the token's key are rotated
    inside the kernel, and key and value are appended to the cache (no separate rope/append launch)."""
    B = _attention_decode_checks(q, k_cache, v_cache, pos, slot, page_table, out, n_q, n_kv, head_dim, cos, sin,
                                 "attention_decode")
    if n_splits > 64:
        raise KernelError("attention_decode: at most 64 splits")
    if n_splits > 1:
        need_f, need_c = attention_decode_scratch(B, n_q, n_kv, head_dim, n_splits)
        _need(scratch, "scratch", torch.float32); _need(counters, "counters", torch.int32)
        if scratch.numel() < need_f or counters.numel() < need_c:
            raise KernelError(f"attention_decode: scratch of {need_f} floats and {need_c} counters needed")
    _check(_fn("decode_ops", "ssb_attention_decode")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(slot), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        c_int(n_splits), _ptr(scratch), _ptr(counters), c_int(1 if pdl else 0), _ptr(cos), _ptr(sin),
        _stream()), "attention_decode")


def attention_decode_chunked_ok(n_seqs: int, n_q: int, n_kv: int, head_dim: int, ldq: int, page_shift: int) -> bool:
    """Whether the tensor-core decode attention takes this case (head sizes 64 and 128, at most 16
    query heads per kv head, 64-token pages, at most 1,024 sequences)."""
    return bool(_fn("decode_ops", "ssb_attention_decode_chunked_ok")(
        c_int(n_seqs), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(ldq), c_int(page_shift)))


_chunked_blocks = {}


def attention_decode_chunked_blocks(n_seqs: int, n_q: int, n_kv: int, head_dim: int, fused: bool) -> int:
    """Blocks of the tensor-core decode attention that the current device holds at once for this case
    (the size of its persistent grid)."""
    key = (torch.cuda.current_device(), min(n_seqs, 1024) > 64, min(n_seqs, 1024) > 256, n_seqs > 512, n_q, n_kv,
           head_dim, bool(fused))
    if key not in _chunked_blocks:
        lib = load_library("decode_ops")
        lib.ssb_attention_decode_chunked_blocks.restype = c_longlong
        _chunked_blocks[key] = int(lib.ssb_attention_decode_chunked_blocks(
            c_int(n_seqs), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(1 if fused else 0)))
    return _chunked_blocks[key]


_chunked_clusters = {}


def attention_decode_chunked_clusters(n_q: int, n_kv: int, head_dim: int, fused: bool, cluster: int) -> int:
    """Thread-block clusters of ``cluster`` (2, 4 or 8) blocks of the tensor-core decode attention that the
    current device holds at once (0: it cannot place one)."""
    key = (torch.cuda.current_device(), n_q, n_kv, head_dim, bool(fused), cluster)
    if key not in _chunked_clusters:
        _chunked_clusters[key] = int(_fn("decode_ops", "ssb_attention_decode_chunked_clusters")(
            c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(1 if fused else 0), c_int(cluster)))
    return _chunked_clusters[key]


def attention_decode_chunked_scratch(n_seqs: int, n_q: int, n_kv: int, head_dim: int, max_chunks: int):
    """(float32 elements of scratch, int32 counters) a launch needs; counters start at zero."""
    lib = load_library("decode_ops")
    lib.ssb_attention_decode_chunked_scratch_floats.restype = c_longlong
    return (int(lib.ssb_attention_decode_chunked_scratch_floats(c_int(n_seqs), c_int(n_q), c_int(head_dim),
                                                                c_int(max_chunks))), n_seqs * n_kv)


def attention_decode_chunked(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                             slot: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                             head_dim: int, page_shift: int, window: Optional[int], scale: float,
                             chunk_pages: int, max_chunks: int, scratch: Optional[torch.Tensor],
                             counters: Optional[torch.Tensor], pdl: bool = False,
                             cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                             cluster: int = 0) -> None:
    """``attention_decode`` on the tensor cores with a persistent grid: every sequence's pages are cut
    into chunks of about ``chunk_pages`` pages (a cut that depends on the sequence alone), a work item
    is (sequence, chunk, kv head), and as many blocks as the device holds at once walk the items.
    ``chunk_pages`` 0: the kernel sizes the chunks itself so that the items about fill those blocks.
    ``max_chunks`` bounds the chunks of one sequence and sizes the scratch
    (:func:`attention_decode_chunked_scratch`); a longer sequence gets ``max_chunks`` larger chunks.
    Pages come in through the TMA unit with bounded waits (:func:`check_device_errors`).
    ``cluster`` 2, 4 or 8: every sequence is cut into that many chunks, the chunks of a (sequence, kv
    head) are the blocks of a thread-block cluster and merge through its shared memory (no scratch);
    for small batches whose blocks all fit the device at once."""
    global _tc_unchecked
    B = _attention_decode_checks(q, k_cache, v_cache, pos, slot, page_table, out, n_q, n_kv, head_dim, cos, sin,
                                 "attention_decode_chunked")
    if chunk_pages < 0 or max_chunks < 1:
        raise KernelError("attention_decode_chunked: chunk_pages must not be negative, max_chunks at least 1")
    if cluster not in (0, 2, 4, 8):
        raise KernelError("attention_decode_chunked: a cluster holds 2, 4 or 8 chunks")
    if max_chunks > 1 and not cluster:
        need_f, need_c = attention_decode_chunked_scratch(B, n_q, n_kv, head_dim, max_chunks)
        _need(scratch, "scratch", torch.float32); _need(counters, "counters", torch.int32)
        if scratch.numel() < need_f or counters.numel() < need_c:
            raise KernelError(f"attention_decode_chunked: scratch of {need_f} floats and {need_c} counters needed")
    _check(_fn("decode_ops", "ssb_attention_decode_chunked")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(slot), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        c_int(chunk_pages), c_int(max_chunks), _ptr(scratch), _ptr(counters), c_int(1 if pdl else 0), _ptr(cos),
        _ptr(sin), c_longlong(k_cache.numel() // head_dim), _ptr(tc_error_word(q.device)), c_int(cluster),
        _stream()), "attention_decode_chunked")
    _tc_unchecked += 1


# ---- prefill GEMM on tcgen05 ---------------------------------------------------------------
TC_STORE, TC_ACCUMULATE, TC_SWIGLU = 0, 1, 2
TC_TILE_PAIR = 512        # ``tile_n`` that asks for 256 x 256 tiles on SM pairs (tcgen05 cta_group::2)
_TC_ERRORS = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue"}
_tc_error_words = {}
_tc_unchecked = 0      # tcgen05 launches since the error words were last read


_after_error = []       # weak references to callables that put scratch back in order after a failed launch


def after_device_error(method) -> None:
    """Register a bound method to be called when a bounded wait is found to have run out, before the
    error is raised: a launch that gave up may have left arrival counters and zero-between-uses
    scratch in a state that later launches would trip over.  Held weakly."""
    import weakref
    _after_error.append(weakref.WeakMethod(method))


def _raise_wait_ran_out(code: int):
    for ref in list(_after_error):
        fn = ref()
        if fn is None:
            _after_error.remove(ref)
        else:
            fn()
    raise KernelError(f"tcgen05 kernel: a bounded wait ran out in {_TC_ERRORS.get(code, code)}; "
                      "the result of that launch is invalid")


def bounded_wait_launches() -> int:
    """Launches since the last look at the error words of kernels whose waits are bounded."""
    return _tc_unchecked


def note_bounded_wait_launches(n: int) -> None:
    """A captured graph that holds ``n`` such launches was replayed: they ran without passing
    through this module, so the error word counts as unread."""
    global _tc_unchecked
    _tc_unchecked += int(n)


def tc_error_word(device) -> torch.Tensor:
    """The device word in which tcgen05 kernels record a wait that ran out (zero = all well)."""
    key = torch.device(device)
    if key not in _tc_error_words:
        _tc_error_words[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _tc_error_words[key]


def check_device_errors(device=None) -> None:
    """Raise if a kernel recorded a bounded wait that ran out.  Reads one word per device, and
    only if a kernel that could have set it was launched since the last look."""
    global _tc_unchecked
    if not _tc_unchecked:
        return
    _tc_unchecked = 0
    for dev, word in list(_tc_error_words.items()):
        if device is not None and torch.device(device) != dev:
            continue
        code = int(word.item())
        if code:
            word.zero_()
            _raise_wait_ran_out(code)


_fetch_buffers = {}


def fetch_with_errors(values: torch.Tensor) -> list:
    """The int32 values of a device tensor as a host list, read in the same wait as the device's
    error word: one synchronisation a step instead of two.  Raises like ``check_device_errors``."""
    global _tc_unchecked
    dev = values.device
    n = values.numel()
    word = _tc_error_words.get(dev) if _tc_unchecked else None
    buf = _fetch_buffers.get(dev)
    if buf is None or buf.numel() < n + 1:
        buf = _fetch_buffers[dev] = torch.empty(max(n + 1, 4097), dtype=torch.int32, pin_memory=True)
    buf[:n].copy_(values.view(-1), non_blocking=True)
    if word is not None:
        buf[n:n + 1].copy_(word, non_blocking=True)
    torch.cuda.current_stream(dev).synchronize()
    out = buf[:n].tolist()
    if word is not None:
        _tc_unchecked = 0
        code = int(buf[n])
        if code:
            word.zero_()
            _raise_wait_ran_out(code)
    return out


class Fetch:
    """An int32 device tensor on its way to the host (:func:`start_fetch`)."""

    __slots__ = ("buf", "n", "event", "with_word", "device")


_fetch_ring = {}


def start_fetch(values: torch.Tensor) -> Fetch:
    """Begin copying the int32 ``values`` (and the device's error word, if a kernel that could set it
    ran since the last look) to pinned host memory on the current stream; nothing waits.  The ring
    holds four copies in flight per device."""
    global _tc_unchecked
    dev = values.device
    n = values.numel()
    ring = _fetch_ring.setdefault(dev, {"bufs": [None] * 4, "turn": 0})
    i = ring["turn"]
    ring["turn"] = (i + 1) % 4
    buf = ring["bufs"][i]
    if buf is None or buf.numel() < n + 1:
        buf = ring["bufs"][i] = torch.empty(max(n + 1, 4097), dtype=torch.int32, pin_memory=True)
    f = Fetch()
    f.buf, f.n, f.device = buf, n, dev
    f.with_word = bool(_tc_unchecked) and dev in _tc_error_words
    buf[:n].copy_(values.view(-1), non_blocking=True)
    if f.with_word:
        buf[n:n + 1].copy_(_tc_error_words[dev], non_blocking=True)
        _tc_unchecked = 0
    f.event = torch.cuda.Event()
    f.event.record()
    return f


def finish_fetch(f: Fetch) -> list:
    """Wait for the copy and return the values; raises like ``check_device_errors``."""
    f.event.synchronize()
    out = f.buf[:f.n].tolist()
    if f.with_word:
        code = int(f.buf[f.n])
        if code:
            _tc_error_words[f.device].zero_()
            _raise_wait_ran_out(code)
    return out


def tc_wait_probe(device="cuda:0") -> None:
    """Launch a block whose only wait can never be satisfied: after about a second it gives up and
    records that in the device's error word, which ``check_device_errors`` then reports."""
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_tc_wait_probe")(_ptr(tc_error_word(device)), _stream()), "tc_wait_probe")


def gemm_tc_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 GEMM takes these operands (else the plain kernel does)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and w.shape[0] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = TC_STORE,
            tile_n: Optional[int] = None, splits: int = 1) -> None:
    """out = a @ w^T on the tensor cores (tcgen05, TMA-fed).  mode: store, add into float32
    ``out``, or SwiGLU over rows of ``w`` that come as [8 gate | 8 up] per 16.  ``splits`` > 1
    (mode accumulate): every tile's K range is cut into that many parts, which add with float atomics."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", None, 2)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if mode == TC_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out):
        raise KernelError(f"gemm_tc: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if tile_n is None:
        tile_n = 256 if N > 128 else 128
    if tile_n == TC_TILE_PAIR and splits != 1:
        raise KernelError("gemm_tc: tiles on SM pairs do not split K")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_gemm_tc")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K), c_int(mode), c_int(tile_n), c_int(splits),
        _ptr(tc_error_word(a.device)), _stream()), "gemm_tc")


def gemm_tc_rope_append(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cos: torch.Tensor,
                        sin: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, page_table: torch.Tensor,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                        page_shift: int, tile_n: int = 256) -> None:
    """The fused query/key/value projection of packed tokens (``w`` = [q; k; v] rows) on tcgen05
    whose epilogue rotates q and k from the float32 sums, writes q (bfloat16) into ``q_out`` and
    k and v into the paged cache entry; nothing else is written.  head_dim 64 or 128, full-width
    rotation, tables [positions, head_dim/2] float32.  Rows with a negative slot are skipped."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(q_out, "q_out", torch.bfloat16, 2)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1); _need(page_table, "page_table", torch.int32, 2)
    _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    M, K = a.shape
    if head_dim not in (64, 128):
        raise KernelError(f"gemm_tc_rope_append: head_dim {head_dim} (64 or 128)")
    if tuple(w.shape) != ((n_q + 2 * n_kv) * head_dim, K) or q_out.shape[0] != M or q_out.shape[1] < n_q * head_dim:
        raise KernelError(f"gemm_tc_rope_append: shapes a{tuple(a.shape)} w{tuple(w.shape)} q_out{tuple(q_out.shape)}")
    if pos.shape[0] != M or slot.shape[0] != M:
        raise KernelError("gemm_tc_rope_append: one position and one slot per row")
    if cos.shape != sin.shape or cos.shape[1] * 2 != head_dim or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError("gemm_tc_rope_append: cos/sin must be [positions, head_dim/2], contiguous")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape \
            or tuple(k_cache.shape[1:]) != (n_kv, 1 << page_shift, head_dim):
        raise KernelError(f"gemm_tc_rope_append: cache shape {tuple(k_cache.shape)}")
    if not gemm_tc_ok(a, w, q_out):
        raise KernelError("gemm_tc_rope_append: operands must be 16-byte aligned with strides in multiples of 8")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_gemm_tc_rope_append")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(q_out), c_int(q_out.stride(0)), c_int(M),
        c_int(K), _ptr(pos), _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache),
        _ptr(cos), _ptr(sin), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(page_shift), c_int(tile_n),
        _ptr(tc_error_word(a.device)), _stream()), "gemm_tc_rope_append")


# ---- prefill attention -------------------------------------------------------------------------
def attention_prefill_ok(q: torch.Tensor, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and head_dim in (64, 128) and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_new: torch.Tensor,
                      seq_start: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                      out: torch.Tensor, max_new: int, n_q: int, n_kv: int, head_dim: int, page_shift: int,
                      window: Optional[int], scale: float) -> None:
    """Causal attention of each sequence's new tokens (packed rows of ``q``) over its cached keys,
    which already include the new ones."""
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    for name, t in (("cu_new", cu_new), ("seq_start", seq_start), ("seq_slot", seq_slot)):
        _need(t, name, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    n_seqs = seq_slot.shape[0]
    if cu_new.shape[0] != n_seqs + 1 or seq_start.shape[0] != n_seqs:
        raise KernelError("attention_prefill: cu_new has one more entry than there are sequences")
    if out.shape[0] != q.shape[0] or out.shape[1] < n_q * head_dim or q.shape[1] < n_q * head_dim:
        raise KernelError("attention_prefill: q/out shapes")
    _check(_fn("prefill_attention", "ssb_attention_prefill")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(cu_new), _ptr(seq_start),
        _ptr(seq_slot), _ptr(page_table), c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)),
        c_int(n_seqs), c_int(max_new), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(page_shift),
        c_int(int(window) if window else 0), c_float(scale), _stream()), "attention_prefill")


def attention_prefill_tc_ok(q: torch.Tensor, out: torch.Tensor, head_dim: int, page_shift: int) -> bool:
    return (q.dtype == torch.bfloat16 and head_dim in (64, 128) and page_shift == 6 and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_new: torch.Tensor,
                         seq_start: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, max_new: int, n_q: int, n_kv: int, head_dim: int, page_shift: int,
                         window: Optional[int], scale: float) -> None:
    """``attention_prefill`` on tcgen05: scores and probabilities in tensor memory, pages by TMA.
    head_dim 64 or 128 and 64-token pages only.  A wait that runs out sets the device's error word
    (``check_device_errors``)."""
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    for name, t in (("cu_new", cu_new), ("seq_start", seq_start), ("seq_slot", seq_slot)):
        _need(t, name, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    n_seqs = seq_slot.shape[0]
    if cu_new.shape[0] != n_seqs + 1 or seq_start.shape[0] != n_seqs:
        raise KernelError("attention_prefill_tc: cu_new has one more entry than there are sequences")
    if out.shape[0] != q.shape[0] or out.shape[1] < n_q * head_dim or q.shape[1] < n_q * head_dim:
        raise KernelError("attention_prefill_tc: q/out shapes")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape \
            or tuple(k_cache.shape[1:]) != (n_kv, 1 << page_shift, head_dim):
        raise KernelError(f"attention_prefill_tc: cache shape {tuple(k_cache.shape)}")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("prefill_attention_tc", "ssb_attention_prefill_tc")(
        _ptr(q), c_int(q.stride(0)), c_int(q.shape[0]), _ptr(k_cache), _ptr(v_cache), c_int(k_cache.shape[0]),
        _ptr(cu_new), _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), c_int(page_table.shape[1]),
        _ptr(out), c_int(out.stride(0)), c_int(n_seqs), c_int(max_new), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        _ptr(tc_error_word(q.device)), _stream()), "attention_prefill_tc")


# ---- decode projections on tcgen05, weights on the M side ------------------------------------------
_sm_counts = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once per device)."""
    dev = torch.cuda.current_device()
    if dev not in _sm_counts:
        _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_counts[dev]


GEMV_TC_MAX_ROWS = 128     # rows of x that gemv_tc takes (the N side of its MMA: 16, 32, 64 or 128)


def gemv_tc_splits(n: int, k: int) -> int:
    """Blocks that share the K range of one 128-row tile of W: up to two blocks per SM in all
    (every SM must pull for the memory system to be busy), at least 4 k-blocks (256 columns) each and
    at most 16 (measured on decode steps of 1B, 3B and 8B sizes: with 8 and 8 the small projections
    of a narrow model filled a third of the SMs, and its steps took 5 to 7 % longer)."""
    tiles = (n + 127) // 128
    return max(1, min(2 * sm_count() // tiles, (k // 64) // 4, 16))


def gemv_tc_scratch(rows: int, n: int, splits: int):
    lib = load_library("gemv_tc")
    lib.ssb_gemv_tc_scratch_floats.restype = c_longlong
    return (int(lib.ssb_gemv_tc_scratch_floats(c_int(rows), c_int(n), c_int(splits))),
            int(lib.ssb_gemv_tc_counters(c_int(n))))


def gemv_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = TC_STORE, splits: int = 1,
            partials: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
            pdl: bool = False) -> None:
    """out = x @ w^T for up to 128 rows with the weights as the M side of tcgen05.mma (they stream
    once, 16 KB a stage).  ``splits`` > 1 shares the K range of a row tile among blocks: store
    and SwiGLU outputs then need ``partials``/``counters`` sized by :func:`gemv_tc_scratch`
    (counters zeroed once) and are summed in a fixed order; mode accumulate adds with float
    atomics instead (no scratch; the last bits may differ between runs)."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", None, 2)
    B, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if mode == TC_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (B, n_out) or B > GEMV_TC_MAX_ROWS:
        raise KernelError(f"gemv_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if splits > 1 and (mode != TC_ACCUMULATE or partials is not None):
        nf, nc = gemv_tc_scratch(B, N, splits)
        _need(partials, "partials", torch.float32); _need(counters, "counters", torch.int32)
        if partials.numel() < nf or counters.numel() < nc:
            raise KernelError(f"gemv_tc: scratch of {nf} floats and {nc} counters needed")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemv_tc", "ssb_gemv_tc")(
        _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(B), c_int(N), c_int(K), c_int(mode), c_int(splits),
        _ptr(partials), _ptr(counters), _ptr(tc_error_word(x.device)), c_int(1 if pdl else 0), _stream()),
        "gemv_tc")


# ---- vector element-wise kernels ------------------------------------------------------------------
def rmsnorm_vec_ok(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    return (out.dtype == torch.bfloat16 and x.dtype == torch.float32 and x.shape[1] % 4 == 0
            and x.shape[1] <= 8192 and x.is_contiguous() and out.is_contiguous()
            and x.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and weight.dtype in _CODES)


def rmsnorm_vec(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """As :func:`rmsnorm` with bfloat16 output, 16-byte loads and the row kept in registers."""
    _need(x, "x", torch.float32, 2); _need(weight, "weight", None, 1); _need(out, "out", torch.bfloat16, 2)
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] != n:
            raise KernelError("rmsnorm_vec: one output row per gathered row")
    elif x.shape[0] != n:
        raise KernelError("rmsnorm_vec: x and out differ in rows")
    if x.shape[1] != out.shape[1] or weight.shape[0] != x.shape[1]:
        raise KernelError("rmsnorm_vec: widths differ")
    _check(_fn("elementwise_ops", "ssb_rmsnorm_vec")(
        _ptr(x), _ptr(rows), _ptr(weight), c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(out), c_int(n),
        c_int(x.shape[1]), c_int(1 if pdl else 0), _stream()), "rmsnorm_vec")


def round_and_clear(sums: torch.Tensor, out: torch.Tensor, pdl: bool = False) -> None:
    """out (bfloat16) = sums (float32, contiguous, same shape) rounded; sums is left zero."""
    _need(sums, "sums", torch.float32, 2); _need(out, "out", torch.bfloat16, 2)
    if sums.shape != out.shape or not sums.is_contiguous() or sums.shape[1] % 8:
        raise KernelError(f"round_and_clear: shapes sums{tuple(sums.shape)} out{tuple(out.shape)}")
    _check(_fn("elementwise_ops", "ssb_round_and_clear")(
        _ptr(sums), _ptr(out), c_int(out.stride(0)), c_int(sums.shape[0]), c_int(sums.shape[1]),
        c_int(1 if pdl else 0), _stream()), "round_and_clear")


def rope_append_vec_ok(qkv: torch.Tensor, cos, head_dim: int, rotary_dim: int, write_cache: bool) -> bool:
    return (qkv.dtype == torch.bfloat16 and cos is not None and write_cache and rotary_dim == head_dim
            and head_dim % 8 == 0 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0)


def rope_append_vec(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
                    slot: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    n_q: int, n_kv: int, head_dim: int, page_shift: int) -> None:
    """As :func:`rope_append` for bfloat16, full-width rotation, with vector loads and stores."""
    _need(qkv, "qkv", torch.bfloat16, 2); _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2); _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    T = qkv.shape[0]
    if qkv.shape[1] < (n_q + 2 * n_kv) * head_dim or pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("rope_append_vec: qkv rows too narrow, or not one position and slot per token")
    if cos.shape != sin.shape or cos.shape[1] * 2 != head_dim or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError("rope_append_vec: cos/sin must be [positions, head_dim/2], contiguous")
    _check(_fn("elementwise_ops", "ssb_rope_append_vec")(
        _ptr(qkv), c_int(qkv.stride(0)), _ptr(cos), _ptr(sin), c_int(cos.shape[0]), _ptr(pos), _ptr(slot),
        _ptr(page_table), c_int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q),
        c_int(n_kv), c_int(head_dim), c_int(page_shift), _stream()), "rope_append_vec")
