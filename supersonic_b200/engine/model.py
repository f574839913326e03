"""The model as the engine runs it: parts built from a :class:`ModelSpec`, a cache, and
one step function.

``step`` takes a batch of sequences that either all start (their prompts, of
unequal lengths, in one step) or all go on by one token.  It runs exactly the
tokens it is given, as one packed batch, against the cache earlier steps left,
appends to the cache, and returns float32 logits at the wanted places.  Nothing
in it depends on the architecture: the order of layers is the spec's schedule.

The reference splits this in two engines, ``prefill_inner`` for a prompt
(crates/runner/src/prefill_engine.rs:974-1382) and ``component_decode_step_4b_impl``
for one token (crates/runner/src/decode_engine.rs:3631-3993), one sequence each.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..config import ModelSpec, load_config, spec_from_config
from ..csrc.kernel_sets import kernel_set_for
from ..parts import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                     BuildContext, WeightAccess, lookup)
from ..weights import WeightStore
from .batch import (NotOnHost, PackedStep, StepBatch, StepEntry, batch_over, decode_pages_bucket, pack_entries,
                    pack_step, plan_chunks)

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {dtype} is not supported (float32 or bfloat16)")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported (float32 or bfloat16)") from None


def _require_cuda(device: torch.device) -> None:
    if device.type != "cuda":
        raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; the engine has no CPU path")
    torch.cuda.set_device(device)


@dataclass
class StepContext:
    batch: StepBatch
    cache: SequenceCache
    kernels: Any
    dtype: torch.dtype
    stage: str = ""            # the part that is running ("embed", "mixer", "feed_forward", "head"): for stage timings


class DecodeGraph:
    """One captured decode step for a fixed number of sequences and key-page bucket.

    Token ids, positions and slots live in a fixed device buffer that each step
    overwrites from pinned host memory; the captured kernels read them from there, so the
    same graph serves any sequences at any positions within the bucket.  The reference has
    no graphs: every op is a host call, several followed by a device synchronise
    (kernels/full_attention_bridge_cuda.cu:1905-1906)."""

    def __init__(self, model: "Model", n_seqs: int, kv_pages: int, pool=None):
        from ..csrc import ops
        B, dev = n_seqs, model.device
        self.n_seqs = B
        # a ring of pinned staging buffers: the host may run several steps ahead of the device
        self.hosts = [torch.zeros(3 * B, dtype=torch.int32).pin_memory() for _ in range(4)]
        self.hosts_np = [h.numpy() for h in self.hosts]     # the same memory, cheap to fill from lists
        self.copied = [None] * len(self.hosts)
        self.turn = 0
        self.ints = torch.zeros(3 * B, dtype=torch.int32, device=dev)
        self.ints[2 * B:] = -1                              # warm-up rows are padding: nothing is written
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.batch = StepBatch(
            n_tokens=B, n_seqs=B, max_new=1, max_total=1, is_decode=True,
            token_ids=self.ints[:B], pos=self.ints[B:2 * B], slot_of_token=self.ints[2 * B:],
            seq_slot=self.ints[2 * B:], seq_start=self.ints[B:2 * B], cu_new=ar, want_rows=ar[:B].clone(),
            n_want=B, kv_pages=kv_pages, host_slots=NotOnHost("host_slots"),
            host_starts=NotOnHost("host_starts"), host_counts=[1] * B)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                       # warm-up outside capture (lazy set-up, attributes)
            model._forward(self.batch)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        before, waits_before = ops.LAUNCHES, ops.bounded_wait_launches()
        with torch.cuda.graph(self.graph, pool=pool):
            self.logits = model._forward(self.batch)
        self.kernels_per_replay = ops.LAUNCHES - before
        # launches of the captured step whose bounded waits can run out: each replay runs them again
        # without passing through their Python faces, so the replay itself must mark the device's
        # error word as unread
        self.waiting_kernels = ops.bounded_wait_launches() - waits_before
        self.pool = self.graph.pool()

    def run(self, tokens, positions, slots) -> torch.Tensor:
        """``tokens``: a host list, or an int32 device tensor (what a sampler just wrote: the step is then
        launched without the host ever seeing them)."""
        i = self.turn
        self.turn = (i + 1) % len(self.hosts)
        if self.copied[i] is not None:
            self.copied[i].synchronize()                    # its last copy has left this buffer
        h = self.hosts[i]
        B = self.n_seqs
        if isinstance(tokens, torch.Tensor):
            self.hosts_np[i][B:] = list(positions) + list(slots)
            self.ints[B:].copy_(h[B:], non_blocking=True)
            self.ints[:B].copy_(tokens.view(-1), non_blocking=True)
        else:
            self.hosts_np[i][:] = list(tokens) + list(positions) + list(slots)     # a numpy view of the pinned buffer
            self.ints.copy_(h, non_blocking=True)
        if self.copied[i] is None:
            self.copied[i] = torch.cuda.Event()
        self.copied[i].record()
        self.graph.replay()
        if self.waiting_kernels:
            from ..csrc import ops
            ops.note_bounded_wait_launches(self.waiting_kernels)
        return self.logits


class PromptGraph:
    """A captured step of prompts (or of pieces of them) for one set of sizes: tokens in all, sequences,
    wanted rows, longest run of new tokens, context bucket.  Recorded the second time a set of sizes
    comes up (the first time runs uncaptured, which also sizes every scratch buffer), then replayed
    for any sequences of those sizes: the step's index arrays are copied into a fixed device buffer
    that the captured kernels read.  What it saves is the host's share of a step, which for prompts of
    a few hundred tokens is larger than the device's.  The reference launches every operation from
    the host, one sequence at a time (crates/runner/src/prefill_engine.rs:974-1382)."""

    def __init__(self, model: "Model", packed: PackedStep, pool=None):
        from ..csrc import ops
        dev = model.device
        n = int(packed.flat.shape[0])
        self.hosts = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.copied = [None, None]
        self.turn = 0
        self.ints = torch.zeros(n, dtype=torch.int32, device=dev)
        self.batch = batch_over(self.ints, packed, captured=True)
        self._load(packed)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        before, waits_before = ops.LAUNCHES, ops.bounded_wait_launches()
        with torch.cuda.graph(self.graph, pool=pool):
            self.logits = model._forward(self.batch)
        self.kernels_per_replay = ops.LAUNCHES - before
        self.waiting_kernels = ops.bounded_wait_launches() - waits_before
        self.pool = self.graph.pool()

    def _load(self, packed: PackedStep) -> None:
        i = self.turn
        self.turn = 1 - i
        if self.copied[i] is not None:
            self.copied[i].synchronize()
        self.hosts[i].numpy()[:] = packed.flat
        self.ints.copy_(self.hosts[i], non_blocking=True)
        if self.copied[i] is None:
            self.copied[i] = torch.cuda.Event()
        self.copied[i].record()

    def run(self, packed: Optional[PackedStep]) -> torch.Tensor:
        """``packed`` None: the inputs were loaded by the constructor (the step that recorded the graph)."""
        if packed is not None:
            self._load(packed)
        self.graph.replay()
        if self.waiting_kernels:
            from ..csrc import ops
            ops.note_bounded_wait_launches(self.waiting_kernels)
        return self.logits


class Model:
    """Parts, cache and step function of one model on one device."""

    def __init__(self, spec: ModelSpec, store: WeightStore, dtype="bfloat16", device="cuda:0",
                 max_tokens: int = 4096, max_seq_tokens: Optional[int] = None,
                 max_slots: Optional[int] = None, kernels: Optional[str] = None, config=None,
                 use_graphs: bool = True, step_token_budget: int = 32768, preflight: bool = True,
                 deterministic: bool = False):
        spec.validate()
        self.spec, self.config = spec, config
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        _require_cuda(self.device)
        self.kernels = kernel_set_for(self.dtype, kernels, deterministic)
        max_seq = min(max_seq_tokens or spec.max_positions, spec.max_positions, max_tokens)
        if int(step_token_budget) < 1:
            raise ValueError("step_token_budget must be at least 1")
        # weights + cache + the largest step's activations against free memory, before anything is loaded
        from . import preflight as _preflight
        self.memory_estimate = (_preflight.check if preflight else _preflight.estimate_only)(
            spec, store, self.dtype, self.device, max_tokens, max_seq, max_slots, int(step_token_budget))
        weights = WeightAccess(store, self.device)
        build = BuildContext(self.device, self.dtype, self.kernels, weights, max_positions=max_seq + 64)

        def part(table, what, ps):
            return lookup(table, ps.kind, what)(ps.params, ps.weights, build)

        self.embedding = part(EMBEDDINGS, "embedding", spec.embedding)
        self.blocks = []
        for b in spec.blocks:
            mixer = part(MIXERS, "mixer", b.mixer)
            ff = part(FEED_FORWARDS, "feed-forward", b.feed_forward)
            n1, n2 = part(NORMS, "norm", b.mixer_norm), part(NORMS, "norm", b.feed_forward_norm)
            pos = part(POSITION_ENCODINGS, "position encoding", b.position) if b.position else None
            self.blocks.append(lookup(BLOCKS, b.kind, "block")(mixer, ff, n1, n2, pos))
        self.final_norm = part(NORMS, "norm", spec.final_norm)
        self.head = part(HEADS, "head", spec.head)
        weights.forget()

        # what each cache entry must hold is asked of the mixer that writes it
        needs: Dict[int, Any] = {}
        for stop in spec.schedule:
            need = self.blocks[stop.layer].mixer.cache_need()
            if stop.writes_cache:
                if stop.cache in needs and needs[stop.cache] != need:
                    raise ValueError(f"cache entry {stop.cache} is written by mixers with different needs")
                needs[stop.cache] = need
            elif needs.get(stop.cache) != need:
                raise ValueError(f"layer {stop.layer} reads cache entry {stop.cache}, whose layout "
                                 f"{needs.get(stop.cache)} is not its own {need}")
        self.cache = SequenceCache({c: n for c, n in needs.items() if n is not None}, max_tokens,
                                   max_seq, self.dtype, self.device, max_slots)
        # a step of more tokens runs as several, chunk by chunk through the cache (``_chunked_step``)
        self.step_token_budget = int(step_token_budget)
        if self.step_token_budget < 1:
            raise ValueError("step_token_budget must be at least 1")
        # decode steps of the serving path replay captured graphs (one per batch size and page bucket),
        # if the kernel set can be captured and no part says that it cannot (``capture_safe = False``:
        # it reads host lists of the batch, or synchronises)
        parts = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            parts += [b] + [p for p in (getattr(b, n, None) for n in ("mixer", "feed_forward", "mixer_norm",
                                                                     "feed_forward_norm", "position")) if p is not None]
        # ``capture_safe``: True (the default), False, or "decode" for a part whose decode steps can be
        # captured but whose prompt steps cannot
        safe = [getattr(p, "capture_safe", True) for p in parts]
        capturable = use_graphs and getattr(self.kernels, "capturable", False)
        self.use_graphs = capturable and all(x is True or x == "decode" for x in safe)
        # prompt steps whose sizes recur are captured too (see PromptGraph)
        self.use_prompt_graphs = capturable and all(x is True for x in safe)
        self.max_prompt_graphs = 32
        self.prompt_graph_max_tokens = 8192
        self._prompt_graphs: Dict[Any, PromptGraph] = {}
        self._prompt_seen: Dict[Any, int] = {}
        self.prompt_graph_replays = 0
        # the last position any position encoding of the model can encode
        limits = [getattr(getattr(b, "position", None), "max_positions", None) for b in self.blocks]
        self.position_limit = min([int(x) for x in limits if x is not None], default=None)
        self._timed = None      # a TimedKernels while stage timing is on
        # NVTX ranges per layer (SSB200_NVTX=1): for a profiler's timeline of uncaptured steps; the reference
        # marks stages with host timers only (crates/runner/src/decode_engine.rs:10157-10162)
        self.nvtx = os.environ.get("SSB200_NVTX", "") not in ("", "0")
        self._graphs: Dict[Any, DecodeGraph] = {}
        self._graph_pool = None
        self.graph_replays = 0
        self.graph_kernels = 0

    # ---- construction from a folder ---------------------------------------------------
    @staticmethod
    def from_dir(model_dir: str, allow_unexpected_tensors: bool = False, **kw) -> "Model":
        """The model class is chosen by config.json's architecture; weights are checked
        against the configuration before anything is built.  Tensors the architecture declares
        as buffers (``ignorable_tensor(name)``) are passed over; any other unexpected tensor is an
        error unless ``allow_unexpected_tensors`` turns it into a warning."""
        config = load_config(model_dir)
        store = WeightStore.from_dir(model_dir)
        store.check(config.tensor_shapes(), ignorable=getattr(config, "ignorable_tensor", None),
                    allow_unexpected=allow_unexpected_tensors)
        return Model(spec_from_config(config), store, config=config, **kw)

    @staticmethod
    def from_config(config, store: WeightStore, **kw) -> "Model":
        store.check(config.tensor_shapes())
        return Model(spec_from_config(config), store, config=config, **kw)

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    # ---- the step ---------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; returns float32 logits ``[wanted, vocab]`` in the order
        of the entries and of their ``want`` (an empty tensor if nothing is wanted)."""
        cache = self.cache
        starts = cache.lengths([e.slot for e in entries])
        if self.use_graphs and self._timed is None \
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._graph_step(entries, starts)
        if sum(len(e.tokens) for e in entries) > self.step_token_budget:
            return self._chunked_step(entries)
        packed = pack_entries(entries, starts, self.spec.vocab_size)
        for e in entries:          # pages a failed step reserved stay with their slots
            cache.reserve(e.slot, len(e.tokens))
        cache.sync()
        logits = self._prompt_step(packed)
        for e in entries:
            cache.advance(e.slot, len(e.tokens))
        return logits

    def _prompt_step(self, packed: PackedStep) -> torch.Tensor:
        """Run a packed step: through its captured graph if these sizes have one, recording one if
        they come up for the second time, else launch by launch."""
        # a captured step keeps its logits and activations for as long as the model lives: only steps
        # that are small enough for the host's share to matter, with few wanted rows, are recorded
        small = packed.n_tokens <= self.prompt_graph_max_tokens and \
            packed.n_want * self.spec.vocab_size * 4 <= (64 << 20)
        if self.use_prompt_graphs and self._timed is None and small:
            key = packed.shape_key
            graph = self._prompt_graphs.get(key)
            if graph is None:
                seen = self._prompt_seen.get(key, 0) + 1
                self._prompt_seen[key] = seen
                if len(self._prompt_seen) > 4096:
                    self._prompt_seen.clear()
                if seen >= 2 and len(self._prompt_graphs) < self.max_prompt_graphs:
                    self._check_positions(packed.max_total)
                    graph = self._prompt_graphs[key] = PromptGraph(self, packed, self._graph_pool)
                    self._graph_pool = graph.pool
                    packed = None                         # its inputs are loaded
            else:
                self._check_positions(packed.max_total)
            if graph is not None:
                self.prompt_graph_replays += 1
                self.graph_kernels += graph.kernels_per_replay
                return graph.run(packed).clone()          # the graph's own buffer is reused by its next replay
        host = torch.from_numpy(packed.flat).pin_memory()
        return self._forward(batch_over(host.to(self.device, non_blocking=True), packed))

    def _check_positions(self, longest: int) -> None:
        """A captured step cannot look at positions on the host (``Rotary.check_range`` sees the sizes
        the graph was recorded with), so the bound is checked before it is replayed."""
        if self.position_limit is not None and longest > self.position_limit:
            raise ValueError(f"a sequence reaches {longest} tokens, beyond the {self.position_limit} "
                             "positions this model encodes")

    def _chunked_step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of more tokens than ``step_token_budget``: the same tokens as several steps, each
        continuing from the cache the one before left.  Bounds the activations a step holds
        (a float32 residual, the query/key/value rows and the feed-forward's inner rows per token)
        whatever the prompts' lengths; the logits are those of the one step, beyond rounding."""
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        counts = [len(e.tokens) for e in entries]
        for e, n in zip(entries, counts):
            if n == 0:
                raise ValueError(f"slot {e.slot}: an entry must bring at least one token")
            bad = [w for w in e.want if not 0 <= w < n]
            if bad:
                raise ValueError(f"slot {e.slot}: wanted place {bad[0]} is outside its {n} tokens")
            toks = np.asarray(e.tokens, dtype=np.int64)
            off = toks[(toks < 0) | (toks >= self.spec.vocab_size)]
            if off.size:
                raise ValueError(f"token ids {off[:8].tolist()} are outside the vocabulary of {self.spec.vocab_size}")
        for e, n in zip(entries, counts):     # all the room first: nothing runs if the step does not fit
            self.cache.reserve(e.slot, n)
        rows = []
        for chunk in plan_chunks(counts, self.step_token_budget):
            piece = [StepEntry(entries[i].slot, entries[i].tokens[lo:hi],
                               [w - lo for w in entries[i].want if lo <= w < hi]) for i, lo, hi in chunk]
            rows.append(self.step(piece))
        return torch.cat(rows) if len(rows) > 1 else rows[0]

    @property
    def feeds_device_tokens(self) -> bool:
        """Whether ``step_ahead`` can run: decode steps replay captured graphs and are not being timed."""
        return self.use_graphs and self._timed is None

    def step_ahead(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One decode step of ``slots`` whose next tokens are the int32 device tensor ``tokens`` (the
        sampler's output of the step before): launched without the host reading them, so that the
        host's share of a step (bookkeeping, the read-back of the tokens) overlaps the device's.
        Returns the logits of every row."""
        if not self.feeds_device_tokens:
            raise RuntimeError("step_ahead needs captured decode steps (the bfloat16 path with graphs on)")
        if tokens.dtype != torch.int32 or tokens.numel() != len(slots) or tokens.device != self.device:
            raise ValueError("step_ahead: one int32 token per slot, on the model's device")
        return self._graph_decode(list(slots), tokens, self.cache.lengths(slots))

    def _graph_step(self, entries, starts) -> torch.Tensor:
        tokens = [int(e.tokens[0]) for e in entries]
        bad = [t for t in tokens if not 0 <= t < self.spec.vocab_size]
        if bad:
            raise ValueError(f"token ids {bad[:8]} are outside the vocabulary of {self.spec.vocab_size}")
        return self._graph_decode([e.slot for e in entries], tokens, starts)

    def _graph_decode(self, slots, tokens, starts) -> torch.Tensor:
        cache = self.cache
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        self._check_positions(max(starts) + 1)
        cache.reserve_each(slots, 1)
        cache.sync()
        key = (len(slots), decode_pages_bucket(max(starts) + 1))
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._graphs[key] = DecodeGraph(self, key[0], key[1], self._graph_pool)
            self._graph_pool = graph.pool
        logits = graph.run(tokens, starts, slots).clone()     # the graph's own buffer is reused next step
        self.graph_replays += 1
        self.graph_kernels += graph.kernels_per_replay
        cache.advance_each(slots, 1)
        return logits

    def time_stages(self, on: bool = True):
        """Switch per-stage timing of the steps that follow on or off (``engine/stage_timings.py``).
        While it is on, steps run uncaptured through a kernel set that brackets every operation with
        CUDA events; ``stage_times()`` returns the milliseconds per stage since it was last asked."""
        from .stage_timings import TimedKernels
        self._timed = TimedKernels(self.kernels) if on else None
        return self._timed

    def stage_times(self):
        return self._timed.collect() if self._timed is not None else {}

    def _forward(self, batch: StepBatch) -> torch.Tensor:
        ctx = StepContext(batch, self.cache, self._timed or self.kernels, self.dtype)
        if self._timed is not None:
            self._timed.ctx = ctx
        ctx.stage = "embed"
        residual = self.embedding(ctx, batch.token_ids)
        if self.nvtx:                                       # a named range per stop of the schedule, for timelines
            for i, stop in enumerate(self.spec.schedule):
                torch.cuda.nvtx.range_push(f"stop {i} layer {stop.layer}")
                self.blocks[stop.layer].forward(ctx, residual, stop.cache, stop.writes_cache)
                torch.cuda.nvtx.range_pop()
        else:
            for stop in self.spec.schedule:
                self.blocks[stop.layer].forward(ctx, residual, stop.cache, stop.writes_cache)
        if batch.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        ctx.stage = "head"
        normed = self.final_norm(ctx, residual, rows=batch.want_rows)
        return self.head(ctx, normed)

    # ---- what a step must read (for rooflines) ------------------------------------------------
    def weight_tensors(self) -> list:
        """Every device tensor the parts that run in a step hold (mixers, feed-forwards, norms, head),
        each storage once: a tied head and a fused view count with the tensor they share.  Position
        tables and the embedding table are left out: a step reads a row of them per token."""
        parts = [self.final_norm, self.head]
        for b in self.blocks:
            parts += [getattr(b, n, None) for n in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")]
        seen, out = set(), []
        for p in parts:
            for v in (vars(p).values() if p is not None and hasattr(p, "__dict__") else ()):
                if isinstance(v, torch.Tensor) and v.device.type == "cuda" and v.dim() >= 1:
                    key = v.untyped_storage().data_ptr()
                    if key not in seen:
                        seen.add(key)
                        out.append(v)
        return out

    def weight_bytes(self) -> int:
        return sum(t.untyped_storage().nbytes() for t in self.weight_tensors())

    def matrix_elements(self) -> int:
        """Elements of the two-dimensional weights a token passes through (the head aside)."""
        head = {t.untyped_storage().data_ptr() for t in vars(self.head).values() if isinstance(t, torch.Tensor)}
        return sum(t.untyped_storage().nbytes() // t.element_size() for t in self.weight_tensors()
                   if t.dim() == 2 and t.untyped_storage().data_ptr() not in head)

    def decode_step_bytes(self, slots) -> int:
        """Bytes one decode step of ``slots`` has to read: every weight once, a row of the embedding
        per sequence, and the keys and values (and fixed state) of those sequences."""
        row = self.spec.hidden_size * torch.empty((), dtype=self.dtype).element_size()
        return self.weight_bytes() + len(slots) * row + sum(self.cache.bytes_read_for(s) for s in slots)

    def check_errors(self) -> None:
        """Raise if a kernel reported a bounded wait that ran out.  Call after results have been
        brought to the host (it reads a device word, which waits for the stream)."""
        from ..csrc import ops
        ops.check_device_errors(self.device)

    def start_fetch(self, values: torch.Tensor):
        """Begin bringing sampled tokens to the host without waiting (``finish_fetch`` waits)."""
        from ..csrc import ops
        return ops.start_fetch(values)

    def finish_fetch(self, handle) -> list:
        from ..csrc import ops
        return ops.finish_fetch(handle)

    def fetch(self, values: torch.Tensor) -> list:
        """Sampled tokens (an int32 device tensor) as a host list; kernel errors are looked at in
        the same wait (see ``check_errors``)."""
        from ..csrc import ops
        if values.device.type != "cuda":
            return values.tolist()
        return ops.fetch_with_errors(values)

    # ---- sequences --------------------------------------------------------------------
    def open_sequence(self, rng_seed: Optional[int] = None) -> int:
        return self.cache.acquire(rng_seed)

    def close_sequence(self, slot: int) -> None:
        self.cache.release(slot)
