"""Registries of parts: mixers, feed-forwards, norms, position encodings, blocks,
embeddings and heads, each from a name to a class.

A :class:`~supersonic_b200.config.base.PartSpec` names its ``kind``; the model
builder looks the class up here and constructs it with
``cls(params, weights, build)``, where ``params`` are the spec's sizes and
constants, ``weights`` maps the part's weight roles to tensor names and
``build`` is the :class:`BuildContext` (device, dtype, kernel set, weight
access).  No part knows which model it is in; adding one is a
``register_*`` call, from anywhere (tests register toy parts this way).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

import torch

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}


def _register(table: Dict[str, type], what: str) -> Callable[[str], Callable[[type], type]]:
    def named(name: str):
        def deco(cls: type) -> type:
            table[name] = cls
            return cls
        return deco
    return named


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def lookup(table: Dict[str, type], kind: str, what: str) -> type:
    try:
        return table[kind]
    except KeyError:
        raise KeyError(f"unknown {what} {kind!r}; registered: {sorted(table)}") from None


class WeightAccess:
    """Tensors by name on the device, converted once per (name, dtype) and shared,
    so a tied head and its embedding are one buffer."""

    def __init__(self, store, device):
        self.store, self.device = store, torch.device(device)
        self._cache: Dict[Any, torch.Tensor] = {}

    def stored(self, name: str, share: bool = False) -> torch.Tensor:
        """As stored: bfloat16 stays bfloat16, 32-bit stays 32-bit."""
        return self.as_dtype(name, None, share)

    def as_dtype(self, name: str, dtype, share: bool = False) -> torch.Tensor:
        """``share=True`` keeps the converted tensor so that a second asker (a tied head)
        gets the same buffer; other tensors belong to the part that asked."""
        key = (name, dtype)
        if key in self._cache:
            return self._cache[key]
        t = self.store.get(name, self.device)
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        if share:
            self._cache[key] = t
        return t

    def forget(self) -> None:
        """Drop the sharing table once the model is built (parts keep what they use)."""
        self._cache.clear()


@dataclass
class BuildContext:
    device: torch.device
    dtype: torch.dtype            # activation and matrix dtype: float32 or bfloat16
    kernels: Any                  # kernel set (plain or fast)
    weights: WeightAccess
    max_positions: int            # positions the cache can hold per sequence
