"""The library's own random numbers for weights: element ``i`` of a tensor is a function of
``(seed, tensor name, i)`` and nothing else.

The same seed therefore names the same model wherever it is made: on the host (NumPy, here),
on the device (``csrc/random_fill.cu``), whole or tensor by tensor, and whatever the torch
build.  The reference has no random weights at all (it loads a checkpoint:
crates/runner/src/llama31_engine.rs:170-287).

A value is ``mean + std * n`` where ``n`` is a sum of twelve 16-bit uniforms, centred and
scaled to variance 1 (an Irwin-Hall sum: close to a normal within +-6 sigma, and made of
integer arithmetic, so every implementation gives the same bits).  See ``random_fill.cu`` for
the recipe step by step.
"""
from __future__ import annotations

from ctypes import c_double, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Sequence

import numpy as np
import torch

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_CHUNK = 1 << 22            # host elements made at a time (bounds the temporaries)


def fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return h


def _mix_int(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    return _mix_int((int(seed) & _MASK) ^ fnv1a64(name))


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _normals(key: int, first: int, count: int) -> np.ndarray:
    """float64 ``n`` of elements first .. first+count-1."""
    with np.errstate(over="ignore"):
        i = np.arange(first, first + count, dtype=np.uint64) * np.uint64(3)
        s = np.zeros(count, dtype=np.int64)
        for j in range(3):
            z = _mix(np.uint64(key) + (i + np.uint64(j + 1)) * np.uint64(_GOLDEN))
            for shift in (0, 16, 32, 48):
                s += ((z >> np.uint64(shift)) & np.uint64(0xFFFF)).astype(np.int64)
    return (2 * s - 12 * 65535).astype(np.float64) * (1.0 / 131072.0)


def fill_host(seed: int, name: str, shape: Sequence[int], mean: float, std: float,
              dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    key = tensor_key(seed, name)
    count = int(np.prod(shape)) if len(shape) else 1
    out = torch.empty(count, dtype=dtype)
    for first in range(0, count, _CHUNK):
        n = min(_CHUNK, count - first)
        v = (np.float64(mean) + np.float64(std) * _normals(key, first, n)).astype(np.float32)
        out[first:first + n] = torch.from_numpy(v).to(dtype)        # round to nearest even
    return out.view(*shape)


def fill_device(seed: int, name: str, shape: Sequence[int], mean: float, std: float, device,
                dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The same tensor made by the CUDA kernel on ``device``."""
    from ..csrc import ops
    out = torch.empty(tuple(shape), dtype=dtype, device=device)
    with torch.cuda.device(out.device):
        ops._check(ops._fn("random_fill", "ssb_random_fill")(
            c_void_p(out.data_ptr()), c_int(ops.dtype_code(dtype)), c_longlong(0), c_longlong(out.numel()),
            c_ulonglong(tensor_key(seed, name)), c_double(mean), c_double(std), ops._stream()), "random_fill")
    return out


def fill(seed: int, name: str, shape: Sequence[int], mean: float, std: float, device="cpu",
         dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    if torch.device(device).type == "cuda":
        return fill_device(seed, name, shape, mean, std, device, dtype)
    return fill_host(seed, name, shape, mean, std, dtype)
