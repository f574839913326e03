"""What one step runs: the tokens it is given, packed, with each token's sequence,
position and cache slot.

A step never pads: the tokens of all sequences lie back to back (``[sum T]``),
so nothing but real tokens is computed and padding cannot change a result.
The reference steps one sequence at a time (``prefill`` for a whole prompt,
``decode_step(token, pos)`` after it: crates/runner/src/decode_engine.rs:10017-10061,
10557-10569); a ragged batch is this engine's own design.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import host


@dataclass
class StepEntry:
    """One sequence's share of a step: its cache slot, its next tokens, and the
    places among these tokens whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class NotOnHost:
    """Stands where a batch has no host-side copy of a field: a captured decode step serves any
    sequences at any positions, so what it knows of them lives in device tensors only
    (``seq_slot``, ``seq_start``, ``pos``, ``slot_of_token``).  Any use raises, so that a part
    which reads host lists cannot silently do nothing inside a captured step; such a part sets
    ``capture_safe = False`` and the model then runs its decode steps uncaptured."""

    def __init__(self, name: str):
        self._name = name

    def _refuse(self, *a, **k):
        raise RuntimeError(f"batch.{self._name} does not exist in a captured decode step: read the device "
                           "tensors of the batch, or set capture_safe = False on the part that needs it")

    __iter__ = __len__ = __getitem__ = __bool__ = __contains__ = _refuse


@dataclass
class StepBatch:
    """The device tensors are the interface every part may rely on; the ``host_*`` lists exist
    only in steps that are not captured (see :class:`NotOnHost`)."""

    n_tokens: int
    n_seqs: int
    max_new: int                   # longest run of new tokens of one sequence
    max_total: int                 # longest sequence after this step
    is_decode: bool                # every sequence brings exactly one token
    token_ids: torch.Tensor        # [T] int32
    pos: torch.Tensor              # [T] int32: position of each token in its sequence
    slot_of_token: torch.Tensor    # [T] int32
    seq_slot: torch.Tensor         # [B] int32
    seq_start: torch.Tensor        # [B] int32: tokens the sequence held before this step
    cu_new: torch.Tensor           # [B+1] int32: where each sequence's new tokens begin
    want_rows: torch.Tensor        # [W] int32: rows of the packed tokens whose logits are wanted
    n_want: int
    kv_pages: int = 1              # pages the longest sequence spans (decode: rounded down to 2^n)
    host_slots: List[int] = field(default_factory=list)
    host_starts: List[int] = field(default_factory=list)
    host_counts: List[int] = field(default_factory=list)


def decode_pages_bucket(longest: int) -> int:
    """Pages (of 64 tokens) spanned by ``longest`` tokens, rounded down to a power of two: kernels size
    their grids from it (a sequence in the bucket spans fewer than twice as many pages), and a captured
    decode step stays valid while the bucket does."""
    return host.decode_pages_bucket(longest)


def plan_chunks(counts: Sequence[int], budget: int) -> List[List[tuple]]:
    """Cut a step of ``counts[i]`` tokens per entry into sub-steps of at most ``budget`` tokens.

    Returns a list of chunks; a chunk is a list of ``(entry, first, end)``: tokens
    ``first .. end - 1`` of that entry.  Entries keep their order, an entry that does not fit what
    is left of a chunk goes on in the next one, and no entry appears twice in a chunk, so a chunk
    is a step of its own whose sequences continue what earlier chunks left in the cache (the
    reference carries a long prompt through its cache in the same way, chunk by chunk:
    crates/runner/src/prefill_engine.rs:1081-1094).  The arithmetic is the host runtime's."""
    return host.plan_chunks(list(counts), budget)


@dataclass
class PackedStep:
    """A step's index arrays as one host array (tokens, positions, slots per token; slot, start per
    sequence; the offsets of the sequences; the wanted rows) and the sizes that cut it up again."""

    flat: np.ndarray               # int32
    n_tokens: int
    n_seqs: int
    n_want: int
    max_new: int
    max_total: int
    slots: List[int]
    starts: List[int]
    counts: List[int]

    @property
    def kv_pages(self) -> int:
        return decode_pages_bucket(self.max_total)

    @property
    def shape_key(self):
        """What a captured prompt step is valid for: kernels size their grids from these."""
        return (self.n_tokens, self.n_seqs, self.n_want, self.max_new, self.kv_pages)


def pack_entries(entries: Sequence[StepEntry], starts: Sequence[int],
                 vocab_size: Optional[int] = None) -> PackedStep:
    """Lay the entries out back to back on the host; every misuse raises before anything runs.  The
    layout and its checks are the host runtime's (``ssb_pack_step``); here the entries' Python lists
    become the arrays it reads."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    slots = [int(e.slot) for e in entries]
    tok_parts = [np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries]
    counts = [int(t.shape[0]) for t in tok_parts]
    want = [int(w) for e in entries for w in e.want]
    flat, (T, B, W, max_new, max_total, _) = host.pack_step(
        slots, [int(s) for s in starts], counts, np.concatenate(tok_parts) if len(tok_parts) > 1 else tok_parts[0],
        [len(e.want) for e in entries], want, vocab_size)
    return PackedStep(flat=flat, n_tokens=T, n_seqs=B, n_want=W, max_new=max_new, max_total=max_total,
                      slots=slots, starts=[int(s) for s in starts], counts=counts)


def batch_over(buf: torch.Tensor, packed: PackedStep, captured: bool = False) -> StepBatch:
    """The :class:`StepBatch` whose device tensors are views of ``buf`` (the packed array on the
    device).  ``captured``: the batch of a step that is recorded once and replayed for other
    sequences of the same sizes, so it carries no host lists."""
    T, B, W = packed.n_tokens, packed.n_seqs, packed.n_want
    o = [0]

    def take(n):
        v = buf[o[0]:o[0] + n]
        o[0] += n
        return v
    token_ids, pos_t, slot_t = take(T), take(T), take(T)
    seq_slot, seq_start, cu_new, want_rows = take(B), take(B), take(B + 1), take(W)
    return StepBatch(
        n_tokens=T, n_seqs=B, max_new=packed.max_new, max_total=packed.max_total, kv_pages=packed.kv_pages,
        is_decode=all(c == 1 for c in packed.counts),
        token_ids=token_ids, pos=pos_t, slot_of_token=slot_t, seq_slot=seq_slot, seq_start=seq_start,
        cu_new=cu_new, want_rows=want_rows, n_want=W,
        host_slots=NotOnHost("host_slots") if captured else packed.slots,
        host_starts=NotOnHost("host_starts") if captured else packed.starts,
        host_counts=NotOnHost("host_counts") if captured else packed.counts)


def pack_step(entries: Sequence[StepEntry], starts: Sequence[int], device,
              vocab_size: Optional[int] = None) -> StepBatch:
    """Lay the entries out back to back and move the index arrays to ``device`` in one copy."""
    packed = pack_entries(entries, starts, vocab_size)
    host = torch.from_numpy(packed.flat)
    dev = torch.device(device)
    if dev.type == "cuda":
        host = host.pin_memory()
    return batch_over(host.to(dev, non_blocking=True), packed)
