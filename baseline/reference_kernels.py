"""DeanoC/SuperSonic's own CUDA kernels, compiled unmodified for sm_100a and called through ctypes.

The reference is a Rust workspace; its model code cannot be built without cargo.  Its kernels
are plain ``.cu`` files with ``extern "C"`` launchers (crates/kernel-ffi/build.rs:284-363 compiles
them with ``nvcc -std=c++17 -O3 --use_fast_math``), so they can stand on their own: this module
copies the three bridge files and their headers into ``baseline/_ref/kernels`` (the installed
reference; not part of the repository), compiles each into a shared library beside them with
the reference's own flags and binds the component launchers.  The persistent "megakernel" entry
points of the same files are never bound: the reference documents that they can hang
(README.md:589-591).

Tests compare these kernels' outputs with the plain implementation's formulas; ``bench.py --impl
reference`` times them per operation.  Every launcher runs on the legacy default stream
(kernels/full_attention_bridge_cuda.cu:118-140), so callers synchronise around a call.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
from ctypes import c_float, c_int, c_size_t, c_uint32, c_void_p
from typing import Dict, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
KERNEL_DIR = os.path.join(REF_DIR, "kernels")
SOURCE_DIR = os.environ.get("SUPERSONIC_REFERENCE", "/root/reference")

# bridge file -> (library name, headers it includes, extra link flags)
BRIDGES = {
    "prefill_helpers_bridge_cuda.cu": ("prefill_helpers", ["prefill_helpers_cuda.cuh"], []),
    "full_attention_bridge_cuda.cu": ("full_attention", ["full_attention_cuda.cuh"], []),
    "full_attention_bridge_4b_cuda.cu": ("full_attention_4b", ["full_attention_4b_cuda.cuh"], ["-lcublas"]),
}
FLAGS = ["-std=c++17", "-O3", "--use_fast_math", "-Xcompiler", "-fPIC", "-shared",
         "-gencode=arch=compute_100a,code=sm_100a"]
DTYPE_F32, DTYPE_BF16 = 1, 2        # the reference's dtype codes (crates/gpu-hal/src/scalar_type.rs:25-32)


class ReferenceUnavailable(RuntimeError):
    pass


def _nvcc() -> Optional[str]:
    for cand in (os.environ.get("SSB200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    return None


def library_path(name: str) -> str:
    return os.path.join(REF_DIR, f"libsupersonic_ref_{name}.so")


def install(verbose: bool = True) -> Dict[str, str]:
    """Copy the bridge sources out of the reference checkout (if it is there) and compile what is
    not compiled yet.  Returns library name -> path; raises :class:`ReferenceUnavailable`."""
    os.makedirs(KERNEL_DIR, exist_ok=True)
    src = os.path.join(SOURCE_DIR, "kernels")
    for bridge, (_, headers, _) in BRIDGES.items():
        for f in [bridge] + headers:
            dst = os.path.join(KERNEL_DIR, f)
            if not os.path.isfile(dst):
                if not os.path.isfile(os.path.join(src, f)):
                    raise ReferenceUnavailable(f"{f} is neither under {KERNEL_DIR} nor under {src}")
                shutil.copyfile(os.path.join(src, f), dst)
    out = {}
    for bridge, (name, _, link) in BRIDGES.items():
        so = library_path(name)
        if not os.path.isfile(so):
            nvcc = _nvcc()
            if nvcc is None:
                raise ReferenceUnavailable("nvcc not found: the reference's kernels cannot be compiled")
            cmd = [nvcc] + FLAGS + ["-I", KERNEL_DIR, os.path.join(KERNEL_DIR, bridge)] + link + ["-o", so + ".tmp"]
            if verbose:
                print(f"[reference] compiling {bridge} for sm_100a ...", file=sys.stderr, flush=True)
            proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if proc.returncode != 0:
                raise ReferenceUnavailable(f"nvcc failed for {bridge}:\n{proc.stdout[-2000:]}")
            os.replace(so + ".tmp", so)
        out[name] = so
    return out


_libs: Dict[str, ctypes.CDLL] = {}


def _lib(name: str) -> ctypes.CDLL:
    if name not in _libs:
        so = library_path(name)
        if not os.path.isfile(so):
            raise ReferenceUnavailable(f"{so} is not built (run: python -m baseline.reference_kernels)")
        try:
            _libs[name] = ctypes.CDLL(so, mode=ctypes.RTLD_LOCAL)
        except OSError as e:
            raise ReferenceUnavailable(f"cannot load {so}: {e}") from None
    return _libs[name]


def available() -> Optional[str]:
    """None if every library loads, else the reason."""
    try:
        for _, (name, _, _) in BRIDGES.items():
            _lib(name)
    except ReferenceUnavailable as e:
        return str(e)
    return None


def _call(lib: str, fn: str, argtypes, *args) -> None:
    f = getattr(_lib(lib), fn)
    f.restype = c_int
    f.argtypes = argtypes
    status = f(*args)
    if status:
        raise RuntimeError(f"reference {fn} returned status {status}")


def _p(t) -> c_void_p:
    return c_void_p(t.data_ptr())


def _sync(t) -> None:
    import torch
    torch.cuda.synchronize(t.device)


# ---- the component launchers (tensors are torch CUDA tensors, bfloat16 unless said otherwise) ----
def rms_norm(x, weight, eps: float, add_unit_offset: bool = False):
    """kernels/full_attention_bridge_cuda.cu:4134 -> full_attention_cuda.cuh:2826-2873.  x [rows, cols]."""
    import torch
    out = torch.empty_like(x)
    _sync(x)
    _call("full_attention", "supersonic_qwen35_hip_rms_norm",
          [c_int, c_size_t, c_size_t, c_size_t, c_float, c_int, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, x.device.index or 0, x.shape[0], x.shape[1], eps, 1 if add_unit_offset else 0,
          _p(x), _p(weight), _p(out))
    _sync(x)
    return out


def apply_rope_prefill(data, cos, sin, first_position: int = 0, rotary_dim: Optional[int] = None):
    """kernels/prefill_helpers_bridge_cuda.cu:620 -> prefill_helpers_cuda.cuh:80-111.  ``data``
    [tokens, heads, head_dim] is rotated in place; row t takes table row ``first_position + t``
    (the caller offsets the table pointers, as crates/runner/src/prefill_engine.rs does)."""
    T, H, D = data.shape
    half = (rotary_dim or D) // 2
    assert cos.shape[1] == half and cos.dtype == data.dtype and cos.is_contiguous() and sin.is_contiguous()
    assert first_position + T <= cos.shape[0]
    off = first_position * half * cos.element_size()
    _sync(data)
    _call("prefill_helpers", "supersonic_qwen35_hip_apply_rope_prefill",
          [c_int, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, data.device.index or 0, T, H, D, half,
          c_void_p(cos.data_ptr() + off), c_void_p(sin.data_ptr() + off), _p(data))
    _sync(data)
    return data


def element_add(lhs, rhs):
    """out = bf16(lhs + rhs), the residual add (kernels/prefill_helpers_bridge_cuda.cu:608 ->
    prefill_helpers_cuda.cuh:60-70)."""
    import torch
    out = torch.empty_like(lhs)
    _sync(lhs)
    _call("prefill_helpers", "supersonic_qwen35_hip_element_add",
          [c_int, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, lhs.device.index or 0, lhs.numel(), _p(lhs), _p(rhs), _p(out))
    _sync(lhs)
    return out


def swiglu_mul(gate, up):
    """kernels/full_attention_bridge_cuda.cu:3147 -> full_attention_cuda.cuh:1995-2010."""
    import torch
    out = torch.empty_like(gate)
    _sync(gate)
    _call("full_attention", "supersonic_qwen35_hip_swiglu_mul",
          [c_int, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, gate.device.index or 0, gate.numel(), _p(gate), _p(up), _p(out))
    _sync(gate)
    return out


def matmul_rhs_transposed(lhs, rhs):
    """out[m, n] = sum_k lhs[m, k] rhs[n, k]: the tiled prompt GEMM,
    kernels/full_attention_bridge_4b_cuda.cu:3597 -> full_attention_4b_cuda.cuh:2671-2743."""
    import torch
    m, k = lhs.shape
    n = rhs.shape[0]
    out = torch.empty((m, n), dtype=lhs.dtype, device=lhs.device)
    _sync(lhs)
    _call("full_attention_4b", "supersonic_qwen35_4b_hip_matmul_rhs_transposed_tiled",
          [c_int, c_size_t, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, lhs.device.index or 0, 1, m, n, k, _p(lhs), _p(rhs), _p(out))
    _sync(lhs)
    return out


def gemv_bf16(x, weight):
    """One row through cuBLAS, the reference's decode projection
    (kernels/full_attention_bridge_4b_cuda.cu:4768-4813).  x [k], weight [n, k] -> [n]."""
    import torch
    n, k = weight.shape
    out = torch.empty(n, dtype=x.dtype, device=x.device)
    _sync(x)
    _call("full_attention_4b", "supersonic_qwen35_4b_cuda_lm_head_bf16_gemm",
          [c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p],
          x.device.index or 0, k, n, _p(x), _p(weight), _p(out))
    _sync(x)
    return out


def attention_prefill(q, k, v, scale: float, seqlen_offset: int = 0):
    """kernels/full_attention_bridge_cuda.cu:1976 -> full_attention_cuda.cuh:360-474.  q [1, nq, T, hd],
    k and v [1, nkv, kv_len, hd] (bfloat16); returns float32 [1, nq, T, hd]."""
    import torch
    _, nq, T, hd = q.shape
    nkv, kv_len = k.shape[1], k.shape[2]
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    _sync(q)
    _call("full_attention", "supersonic_qwen35_hip_full_attention_prefill",
          [c_int, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_float,
           c_size_t, c_void_p, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, q.device.index or 0, 1, nq, nkv, T, kv_len, hd, nq // nkv, scale, seqlen_offset,
          _p(q), _p(k), _p(v), _p(out))
    _sync(q)
    return out


def attention_decode(q, k, v, scale: float, kv_len: int):
    """One query token over ``kv_len`` keys of a cache with room for ``k.shape[2]``:
    kernels/full_attention_bridge_cuda.cu:2094 -> full_attention_cuda.cuh:578-679.  q [1, nq, hd],
    k and v [1, nkv, capacity, hd]; returns bfloat16 [1, nq, hd]."""
    import torch
    _, nq, hd = q.shape
    nkv, cap = k.shape[1], k.shape[2]
    out = torch.empty_like(q)
    _sync(q)
    _call("full_attention", "supersonic_qwen35_hip_full_attention_decode_flat_strided",
          [c_int, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_float,
           c_void_p, c_void_p, c_void_p, c_void_p],
          DTYPE_BF16, q.device.index or 0, 1, nq, nkv, kv_len, cap, hd, nq // nkv, scale,
          _p(q), _p(k), _p(v), _p(out))
    _sync(q)
    return out


def lm_head_argmax(hidden, weight, f32_logits: bool = False) -> int:
    """The fused head + greedy pick (kernels/prefill_helpers_bridge_cuda.cu:812/834 -> 289-359):
    each logit rounded to bfloat16 before comparison unless ``f32_logits``; ties go to the lowest index."""
    import torch
    vocab, hdim = weight.shape
    vals = torch.empty(512, dtype=torch.float32, device=hidden.device)
    idxs = torch.empty(512, dtype=torch.int32, device=hidden.device)
    out = torch.zeros(1, dtype=torch.int32, device=hidden.device)
    _sync(hidden)
    _call("prefill_helpers", "supersonic_qwen35_cuda_lm_head_argmax_bf16" + ("_f32accum" if f32_logits else ""),
          [c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
          hidden.device.index or 0, hdim, vocab, _p(hidden), _p(weight), _p(vals), _p(idxs), _p(out))
    _sync(hidden)
    return int(out.item())


def target_nll(logits, targets):
    """Negative log-likelihood of ``targets`` (int32 [rows]) under bfloat16 ``logits`` [rows, vocab]:
    kernels/prefill_helpers_bridge_cuda.cu:780 -> 405-463.  Returns float32 [rows]."""
    import torch
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _sync(logits)
    _call("prefill_helpers", "supersonic_qwen35_cuda_target_nll_bf16",
          [c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p],
          logits.device.index or 0, rows, vocab, _p(logits), _p(targets), _p(out))
    _sync(logits)
    return out


if __name__ == "__main__":
    for lib_name, path in install().items():
        print("built", lib_name, path)
