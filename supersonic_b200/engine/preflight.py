"""Will the model fit?  Asked before a byte of it is on the device.

The reference estimates ``fixed + kv_bytes_per_token * context`` against the card's memory
before it loads anything and prints a ``[vram]`` line (crates/runner/src/llama31_engine.rs:898-928;
the per-model ``fixed_bytes`` come from a table, crates/runner/src/registry.rs:773-785).  Here the
three terms are computed from the model's description, so they hold for any architecture that
is registered:

* weights: every tensor the parts name, in the dtype the path keeps it in;
* cache: what the mixers say they need per cache entry (``cache_need_from(params)``), for the
  pages, tables and per-sequence state of :class:`SequenceCache`;
* workspace: the activations of the largest step (``step_token_budget`` tokens: float32 residual,
  normed copy, and what each part says it holds per token, ``activation_elements(params)``) and
  the logits of a decode step.

A mixer or feed-forward that offers neither hook is counted with a default; the cache checks
itself again when it is built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..cache import SequenceCache
from ..parts import FEED_FORWARDS, MIXERS, lookup

GIB = float(1 << 30)


class MemoryPreflightError(RuntimeError):
    """The device cannot hold the model with the cache that was asked for."""


@dataclass
class MemoryEstimate:
    weights: int
    cache: int
    workspace: int
    free: Optional[int] = None
    total: Optional[int] = None

    @property
    def needed(self) -> int:
        return self.weights + self.cache + self.workspace

    def line(self, max_tokens: int) -> str:
        s = (f"[vram] estimated={self.needed / GIB:.2f}GiB (weights={self.weights / GIB:.2f}GiB + "
             f"kv_cache={self.cache / GIB:.2f}GiB for {max_tokens}tok + workspace={self.workspace / GIB:.2f}GiB)")
        if self.free is not None:
            s += f" available={self.free / GIB:.1f}GiB of {self.total / GIB:.1f}GiB"
        return s


def _part_specs(spec):
    yield spec.embedding
    for b in spec.blocks:
        for p in (b.mixer, b.feed_forward, b.mixer_norm, b.feed_forward_norm, b.position):
            if p is not None:
                yield p
    yield spec.final_norm
    yield spec.head


def weight_bytes(spec, store, dtype: torch.dtype) -> int:
    """Matrices are kept in ``dtype``; vectors (norm weights) as stored.  A tensor two parts name
    (a tied head) is counted once."""
    item = torch.empty((), dtype=dtype).element_size()
    names = {n for p in _part_specs(spec) for n in p.weights.values()}
    total = 0
    for n in names:
        if n not in store:
            continue                       # the weight check reports it; nothing to count
        shape = store.shape(n)
        numel = 1
        for d in shape:
            numel *= int(d)
        stored = torch.empty((), dtype=store.stored_dtype(n)).element_size()
        total += numel * (item if len(shape) >= 2 else stored)
    return total


def cache_needs(spec) -> Dict[int, object]:
    needs: Dict[int, object] = {}
    for stop in spec.schedule:
        if not stop.writes_cache:
            continue
        ps = spec.blocks[stop.layer].mixer
        hook = getattr(lookup(MIXERS, ps.kind, "mixer"), "cache_need_from", None)
        if hook is not None:
            need = hook(ps.params)
            if need is not None:
                needs[stop.cache] = need
    return needs


def workspace_bytes(spec, dtype: torch.dtype, step_tokens: int, decode_rows: int) -> int:
    item = torch.empty((), dtype=dtype).element_size()
    widest = 0
    for b in spec.blocks:
        here = 0
        for ps, table, what in ((b.mixer, MIXERS, "mixer"), (b.feed_forward, FEED_FORWARDS, "feed-forward")):
            hook = getattr(lookup(table, ps.kind, what), "activation_elements", None)
            here = max(here, int(hook(ps.params)) if hook is not None else 4 * spec.hidden_size)
        widest = max(widest, here)
    per_token = 4 * spec.hidden_size + item * (2 * spec.hidden_size + widest)
    return step_tokens * per_token + 2 * decode_rows * spec.vocab_size * 4


def estimate(spec, store, dtype: torch.dtype, max_tokens: int, max_seq_tokens: int,
             max_slots: Optional[int], step_token_budget: int) -> MemoryEstimate:
    from ..cache.sequence_cache import pages_for
    slots = max_slots if max_slots is not None else min(pages_for(max_tokens), 4096)
    return MemoryEstimate(
        weights=weight_bytes(spec, store, dtype),
        cache=SequenceCache.bytes_needed(cache_needs(spec), max_tokens, max_seq_tokens, dtype, max_slots),
        workspace=workspace_bytes(spec, dtype, min(step_token_budget, max_tokens), min(slots, 256)))


def check(spec, store, dtype, device, max_tokens, max_seq_tokens, max_slots, step_token_budget) -> MemoryEstimate:
    """Estimate, compare with what the device has free, raise :class:`MemoryPreflightError`."""
    est = estimate(spec, store, dtype, max_tokens, max_seq_tokens, max_slots, step_token_budget)
    device = torch.device(device)
    if device.type == "cuda":
        free, total = torch.cuda.mem_get_info(device)
        free += torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        est.free, est.total = int(free), int(total)
        if est.needed > free:
            raise MemoryPreflightError(
                est.line(max_tokens) + f": {est.needed / GIB:.2f} GiB do not fit; nothing was loaded.  Ask for "
                "fewer tokens (context size x batch size, or max_tokens)")
    return est


def estimate_only(spec, store, dtype, device, max_tokens, max_seq_tokens, max_slots, step_token_budget) -> MemoryEstimate:
    return estimate(spec, store, dtype, max_tokens, max_seq_tokens, max_slots, step_token_budget)
