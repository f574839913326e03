"""Weights by tensor name, from a model folder or from a seed.

The reference loads each tensor by its stored name with no renaming, splitting
or fusing and reports the first miss as ``load <name>: tensor not found``
(crates/runner/src/llama31_engine.rs:170-287; crates/qwen35/src/loader.rs:142-159).
Here the whole folder is checked against the configuration first, and one
error lists everything that is missing, unexpected or of the wrong shape.

Storage rule: 16-bit floating tensors are kept as bfloat16 (float16 is converted
once), a tensor stored in 32 bits stays 32-bit, integer tables become int32.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from . import random_fill
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


class WeightError(RuntimeError):
    """Missing, unexpected or misshapen tensors; ``missing``/``unexpected``/``wrong_shape``
    hold the lists that the message prints."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, List[int], List[int]]],
                 wrong_dtype: List[Tuple[str, str]] = ()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"weights in {where} do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {want}, found {got}")
        for name, got in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is {got}")
        super().__init__("\n".join(lines))


def _storage_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype in (torch.int64, torch.uint8):
        return t.to(torch.int32)
    return t            # bfloat16, float32, int32 stay as stored


class WeightStore:
    """Name -> tensor.  Sources: a folder of safetensors, or a dict already in memory."""

    def __init__(self, tensors: Dict[str, object], where: str):
        self._tensors = tensors        # name -> torch.Tensor or (SafetensorsFile, name)
        self.where = where

    # ---- sources ----------------------------------------------------------
    @staticmethod
    def from_dir(model_dir: str) -> "WeightStore":
        """Single ``model.safetensors``, the ``-00001-of-00001`` spelling, or shards listed
        by ``model.safetensors.index.json`` (the three cases of loader.rs:65-139)."""
        single = os.path.join(model_dir, "model.safetensors")
        alt = os.path.join(model_dir, "model.safetensors-00001-of-00001.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        tensors: Dict[str, object] = {}
        if os.path.isfile(single) or os.path.isfile(alt):
            f = SafetensorsFile(single if os.path.isfile(single) else alt)
            for n in f.names():
                tensors[n] = (f, n)
        elif os.path.isfile(index):
            try:
                with open(index, "r", encoding="utf-8") as fh:
                    weight_map = json.load(fh)["weight_map"]
            except (OSError, KeyError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{index}: cannot read weight_map: {e}") from None
            files: Dict[str, SafetensorsFile] = {}
            for name, shard in weight_map.items():
                if shard not in files:
                    files[shard] = SafetensorsFile(os.path.join(model_dir, shard))
                if name not in files[shard].names():
                    raise SafetensorsError(f"{index} places {name} in {shard}, which lacks it")
                tensors[name] = (files[shard], name)
        else:
            raise SafetensorsError(f"no model.safetensors or model.safetensors.index.json in {model_dir}")
        return WeightStore(tensors, model_dir)

    @staticmethod
    def from_tensors(tensors: Dict[str, torch.Tensor], where: str = "memory") -> "WeightStore":
        return WeightStore(dict(tensors), where)

    # ---- access -----------------------------------------------------------
    def names(self) -> List[str]:
        return list(self._tensors)

    def __contains__(self, name: str) -> bool:
        return name in self._tensors

    def shape(self, name: str) -> List[int]:
        t = self._tensors[name]
        return t[0].shape(t[1]) if isinstance(t, tuple) else list(t.shape)

    def stored_dtype(self, name: str) -> torch.dtype:
        t = self._tensors[name]
        return t[0].dtype(t[1]) if isinstance(t, tuple) else t.dtype

    def check(self, expected: Dict[str, List[int]], ignorable=None, allow_unexpected: bool = False) -> None:
        """Raise one :class:`WeightError` listing every mismatch with ``expected``.  ``ignorable(name)``
        names stored tensors that are no parameters (buffers some exporters write, such as
        ``rotary_emb.inv_freq``): they are passed over.  ``allow_unexpected``: other unexpected
        tensors are reported with a warning instead of the error (the reference never looks at
        tensors it does not ask for: crates/qwen35/src/loader.rs:142-159)."""
        missing = [n for n in expected if n not in self._tensors]
        unexpected = [n for n in self._tensors if n not in expected and not (ignorable and ignorable(n))]
        if unexpected and allow_unexpected:
            import warnings
            warnings.warn(f"weights in {self.where}: {len(unexpected)} tensors the configuration does not "
                          f"name are ignored: {', '.join(unexpected[:8])}{' ...' if len(unexpected) > 8 else ''}")
            unexpected = []
        wrong_shape, wrong_dtype = [], []
        for n, want in expected.items():
            if n in self._tensors:
                got = self.shape(n)
                if list(got) != list(want):
                    wrong_shape.append((n, list(want), list(got)))
                dt = self.stored_dtype(n)
                if dt not in (torch.bfloat16, torch.float16, torch.float32):
                    wrong_dtype.append((n, str(dt)))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightError(self.where, missing, unexpected, wrong_shape, wrong_dtype)

    def get(self, name: str, device: Optional[torch.device] = None) -> torch.Tensor:
        """The tensor in its storage dtype, on ``device`` (CPU if None)."""
        if name not in self._tensors:
            raise WeightError(self.where, [name], [], [])
        t = self._tensors[name]
        if isinstance(t, tuple):
            t = t[0].tensor(t[1])
        t = _storage_dtype(t)
        if device is not None and t.device != torch.device(device):
            if t.device.type == "cpu" and not t.is_pinned():
                t = t.clone()          # off the read-only map before the copy engine sees it
            t = t.to(device, non_blocking=False)
        return t


# ---- random weights -----------------------------------------------------------
def random_tensor(config, seed: int, name: str, device: str = "cpu", std: float = 0.02,
                  norm_jitter: float = 0.1) -> torch.Tensor:
    """One seeded tensor by name, in bfloat16: matrices and embeddings N(0, std), norm weights
    1 + N(0, norm_jitter).  Its values depend on (seed, name, element index) alone: the same on the
    host and on the device, whole or in pieces (see ``random_fill``)."""
    shape = config.tensor_shapes()[name]
    is_norm = getattr(config, "is_norm_tensor", lambda n: len(shape) == 1)
    if is_norm(name):
        return random_fill.fill(seed, name, shape, 1.0, norm_jitter, device)
    return random_fill.fill(seed, name, shape, 0.0, std, device)


def random_tensors(config, seed: int, device: str = "cpu", std: float = 0.02,
                   norm_jitter: float = 0.1) -> Iterator[Tuple[str, torch.Tensor]]:
    """Seeded tensors for every name the configuration asks for (:func:`random_tensor`)."""
    for name in config.tensor_shapes():
        yield name, random_tensor(config, seed, name, device, std, norm_jitter)


class RandomWeightStore(WeightStore):
    """Random weights made on ``device`` when a tensor is asked for, never all at once."""

    def __init__(self, config, seed: int, device: str = "cpu", std: float = 0.02, norm_jitter: float = 0.1):
        self._shapes = {n: list(s) for n, s in config.tensor_shapes().items()}
        self._args = (config, seed, str(device), std, norm_jitter)
        super().__init__({n: None for n in self._shapes}, f"random(seed={seed})")

    def shape(self, name: str) -> List[int]:
        return list(self._shapes[name])

    def stored_dtype(self, name: str) -> torch.dtype:
        return torch.bfloat16

    def get(self, name: str, device: Optional[torch.device] = None) -> torch.Tensor:
        if name not in self._shapes:
            raise WeightError(self.where, [name], [], [])
        config, seed, made_on, std, jitter = self._args
        t = random_tensor(config, seed, name, made_on, std, jitter)
        return t if device is None or t.device == torch.device(device) else t.to(device)


def random_store(config, seed: int, device: str = "cpu", std: float = 0.02,
                 norm_jitter: float = 0.1) -> WeightStore:
    """Random weights held in memory (on ``device``): no folder is written."""
    return WeightStore.from_tensors(
        dict(random_tensors(config, seed, device, std, norm_jitter)), f"random(seed={seed})")


def write_model_folder(config, seed: int, model_dir: str, std: float = 0.02,
                       norm_jitter: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` of a random model; returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
        f.write("\n")
    entries = [(n, torch.bfloat16, list(s)) for n, s in config.tensor_shapes().items()]
    write_safetensors(os.path.join(model_dir, "model.safetensors"), entries,
                      random_tensors(config, seed, "cpu", std, norm_jitter),
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
