"""Minimal reader and writer of the safetensors container.

File layout: an 8-byte little-endian header length, that many bytes of JSON
(``name -> {dtype, shape, data_offsets}`` plus an optional ``__metadata__``),
then the raw little-endian tensor data.  The reference reads the same files
through the ``safetensors`` crate over an mmap (crates/qwen35/src/loader.rs:65-139);
this is an own parser over ``mmap`` so that nothing but the file format is shared.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``.safetensors`` file, mapped read-only; tensors are views into the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"open {path}: {e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + hlen
        self._entries: Dict[str, Tuple[str, List[int], int, int]] = {}
        for name, info in header.items():
            try:
                dtype, shape = info["dtype"], [int(s) for s in info["shape"]]
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                n *= s
            if end - begin != n * _DTYPES[dtype][1] or begin < 0 or self._data_start + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ({dtype} {shape}) does not match its "
                    f"data_offsets [{begin}, {end}) in a file of {size} bytes")
            self._entries[name] = (dtype, shape, begin, end)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> List[int]:
        return list(self._entries[name][1])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only: clone or copy before writing)."""
        dtype, shape, begin, end = self._entries[name]
        tdtype = _DTYPES[dtype][0]
        if end == begin:
            return torch.empty(shape, dtype=tdtype)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the map is read-only on purpose
            t = torch.frombuffer(buf, dtype=tdtype)
        return t.reshape(shape)


def write_safetensors(path: str, entries: List[Tuple[str, torch.dtype, List[int]]],
                      tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Write ``entries`` (name, dtype, shape: known up front, so the header can be
    written first) and then stream the tensors, which must arrive in that order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    for name, dtype, shape in entries:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        it = iter(tensors)
        for name, dtype, shape in entries:
            got_name, t = next(it)
            if got_name != name or t.dtype != dtype or list(t.shape) != list(shape):
                raise SafetensorsError(f"write {path}: expected {name} {dtype} {shape}, got "
                                       f"{got_name} {t.dtype} {list(t.shape)}")
            t = t.detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
