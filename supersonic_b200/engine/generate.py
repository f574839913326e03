"""The generation loop above the step function.

Requests are served in batches that start together: all prompts of a batch, of unequal
lengths, in one step; then one token per live sequence per step.  A sequence ends at
a stop token or at its token budget, leaves the batch and gives its slot back; the
step shrinks.  No request joins a running batch; the next batch starts when the
current one is done, in slots that were used before.

Per sequence this is the reference's loop (crates/runner/src/llama31_engine.rs:1075-1551):
the first token is sampled from the prompt's last logits; a stop token is appended
to the output before the loop sees it; ``max_new_tokens == 0`` still runs the prompt.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from .. import host
from ..sampling import Sampler, SamplingParams, request_seed
from .batch import StepEntry


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = "length"         # "stop" (a stop token) or "length" (the budget)
    prompt_tokens: int = 0


@dataclass
class RunStats:
    """Host-side account of a ``generate`` call: prompt steps (one per batch) and decode steps, with the
    wall time from a step's start to its tokens being on the host.  The reference prints the same
    split as ``[prefill]`` and ``[result]`` (crates/runner/src/llama31_engine.rs:1083-1087, 1564-1598)."""

    prefill_steps: int = 0
    prefill_tokens: int = 0
    prefill_s: float = 0.0
    decode_steps: int = 0
    decode_tokens: int = 0
    decode_s: float = 0.0


def finished(token: int, n_generated: int, max_new_tokens: int, stop_ids) -> Optional[str]:
    """Why a sequence ends after producing ``token`` as its ``n_generated``-th, or None."""
    return host.finished(token, n_generated, max_new_tokens, stop_ids)


def plan_batch(waiting: Sequence[int], prompt_lens: Sequence[int], max_new_tokens: int,
               free_tokens: int, free_slots: int, page_tokens: int,
               batch_size: Optional[int]) -> List[int]:
    """The next batch: requests in arrival order while their prompts plus budgets fit
    the free pages and slots (each sequence's need rounded up to whole pages)."""
    n = host.plan_batch([prompt_lens[r] for r in waiting], max_new_tokens, free_tokens, free_slots,
                        page_tokens, batch_size)
    return list(waiting[:n])


class Generator:
    """Drives ``model.step`` for whole requests.  ``model`` needs ``step``, ``open_sequence``,
    ``close_sequence``, ``cache`` (``free_tokens``, ``slots.n_free``, ``max_seq_tokens``),
    ``spec.stop_token_ids`` and ``device``; ``sampler`` maps logits and slots to tokens."""

    def __init__(self, model, sampler: Optional[Callable] = None):
        self.model = model
        self.sampler = sampler or Sampler(model.kernels, model.cache.rng_state)
        self.steps_run = 0
        self.stats = RunStats()
        self.stage_timings = None          # {"prefill": StageTimings, "decode": StageTimings} while timing is on

    def time_stages(self, on: bool = True) -> None:
        """Per-stage device timings of the steps that follow (``engine/stage_timings.py``): timed steps
        run uncaptured, operation by operation, so they are slower than untimed ones."""
        from .stage_timings import StageTimings
        self.model.time_stages(on)
        self.stage_timings = {"prefill": StageTimings(), "decode": StageTimings()} if on else None

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 8,
                 sampling: SamplingParams = SamplingParams(), stop_token_ids=None,
                 ignore_eos: bool = False, include_stop_token: bool = True,
                 batch_size: Optional[int] = None,
                 on_step: Optional[Callable] = None) -> List[GenerationResult]:
        from ..cache import PAGE_TOKENS
        model, cache = self.model, self.model.cache
        stop_ids = frozenset() if ignore_eos else frozenset(
            model.spec.stop_token_ids if stop_token_ids is None else stop_token_ids)
        prompts = [list(p) for p in prompts]
        for i, p in enumerate(prompts):
            if not p:
                raise ValueError(f"prompt {i} is empty")
            if len(p) + max_new_tokens > cache.max_seq_tokens:
                raise ValueError(f"prompt {i}: {len(p)} tokens plus {max_new_tokens} new ones exceed "
                                 f"the {cache.max_seq_tokens} a sequence may hold")
        results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
        waiting = list(range(len(prompts)))
        lens = [len(p) for p in prompts]
        while waiting:
            batch = plan_batch(waiting, lens, max_new_tokens, cache.free_tokens(), cache.slots.n_free,
                               PAGE_TOKENS, batch_size)
            if not batch:
                raise RuntimeError(f"request {waiting[0]} ({lens[waiting[0]]} prompt tokens) does not "
                                   f"fit the cache even when it is empty of other requests")
            waiting = waiting[len(batch):]
            self._run_batch(batch, prompts, results, max_new_tokens, sampling, stop_ids,
                            include_stop_token, on_step)
        return results

    def _run_batch(self, batch, prompts, results, max_new_tokens, sampling, stop_ids,
                   include_stop_token, on_step):
        """One batch from its prompts to its last token.  A model that can take a step's tokens from
        the device (``feeds_device_tokens``, ``step_ahead``) is driven one step ahead of the host."""
        if max_new_tokens > 1 and self.stage_timings is None and getattr(self.model, "feeds_device_tokens", False):
            return self._run_batch_ahead(batch, prompts, results, max_new_tokens, sampling, stop_ids,
                                         include_stop_token, on_step)
        model = self.model
        slot_of = {r: model.open_sequence(request_seed(sampling.sampling_seed, r)) for r in batch}
        live = list(batch)
        try:
            entries = [StepEntry(slot_of[r], prompts[r], [len(prompts[r]) - 1]) for r in live]
            slots = None
            first = True
            while live:
                t0 = time.perf_counter()
                n_step_tokens = sum(len(e.tokens) for e in entries)
                logits = model.step(entries)
                self.steps_run += 1
                if max_new_tokens <= 0:
                    if getattr(getattr(model, "device", None), "type", "") == "cuda":
                        torch.cuda.synchronize(model.device)     # nothing is fetched: wait for the prompt step itself
                    self._account(first, n_step_tokens, time.perf_counter() - t0, None)
                    break
                if slots is None:                        # the live set changed (or this is the first step)
                    slots = torch.tensor([slot_of[r] for r in live], dtype=torch.int32).to(
                        logits.device, non_blocking=True)
                timed = self.stage_timings is not None
                if timed:
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                    ev[0].record()
                sampled = self.sampler(logits, slots, sampling)
                if timed:
                    ev[1].record()
                if hasattr(model, "fetch"):
                    tokens = model.fetch(sampled)        # kernel errors are looked at in the same wait
                else:
                    tokens = sampled.to("cpu").tolist()
                self._account(first, n_step_tokens, time.perf_counter() - t0, ev if timed else None)
                first = False
                if on_step:
                    on_step(live, tokens)
                still, entries = [], []
                for r, tok in zip(live, tokens):
                    res = results[r]
                    why = finished(tok, len(res.tokens) + 1, max_new_tokens, stop_ids)
                    if why != "stop" or include_stop_token:
                        res.tokens.append(tok)
                    if why:
                        res.finish_reason = why
                        model.close_sequence(slot_of.pop(r))
                    else:
                        still.append(r)
                        entries.append(StepEntry(slot_of[r], [tok], [0]))
                if len(still) != len(live):
                    slots = None
                live = still
        finally:
            for slot in slot_of.values():
                model.close_sequence(slot)

    def _run_batch_ahead(self, batch, prompts, results, max_new_tokens, sampling, stop_ids,
                         include_stop_token, on_step):
        """The same batch with the device kept one step ahead: step k + 1 is launched from the tokens
        step k sampled while those are still on their way to the host; the host then reads them,
        applies the stop rules and prepares step k + 2.  A sequence that ends at its token budget is
        known beforehand and is not stepped again; one that ends at a stop token has been stepped once
        more than needed by then: that step's token is dropped (it wrote one key and value into a slot
        that is given back right after)."""
        model = self.model
        slot_of = {r: model.open_sequence(request_seed(sampling.sampling_seed, r)) for r in batch}
        device = model.device

        def slots_tensor(rows):
            return torch.tensor([slot_of[r] for r in rows], dtype=torch.int32).to(device, non_blocking=True)
        try:
            rows = list(batch)                           # the requests whose tokens ``sampled`` holds, row by row
            last = time.perf_counter()
            logits = model.step([StepEntry(slot_of[r], prompts[r], [len(prompts[r]) - 1]) for r in rows])
            self.steps_run += 1
            n_step_tokens = sum(len(prompts[r]) for r in rows)
            slots = slots_tensor(rows)
            sampled = self.sampler(logits, slots, sampling)
            handle = model.start_fetch(sampled)
            first = True
            while True:
                # whoever has budget for more than the token that is on its way is stepped again now
                ahead = [r for r in rows if r in slot_of and len(results[r].tokens) + 1 < max_new_tokens]
                if ahead:
                    if ahead == rows:
                        fed = sampled
                    else:
                        at = {r: i for i, r in enumerate(rows)}
                        index = torch.tensor([at[r] for r in ahead], dtype=torch.int64).to(device, non_blocking=True)
                        fed = sampled.index_select(0, index)
                        slots = slots_tensor(ahead)
                    logits = model.step_ahead([slot_of[r] for r in ahead], fed)
                    self.steps_run += 1
                    sampled_ahead = self.sampler(logits, slots, sampling)
                    handle_ahead = model.start_fetch(sampled_ahead)
                tokens = model.finish_fetch(handle)      # kernel errors are looked at in the same wait
                now = time.perf_counter()
                self._account(first, n_step_tokens, now - last, None)
                last, first = now, False
                alive = [(r, t) for r, t in zip(rows, tokens) if r in slot_of]     # not: ended a step ago at a stop token
                if on_step:
                    on_step([r for r, _ in alive], [t for _, t in alive])
                for r, tok in alive:
                    res = results[r]
                    why = finished(tok, len(res.tokens) + 1, max_new_tokens, stop_ids)
                    if why != "stop" or include_stop_token:
                        res.tokens.append(tok)
                    if why:
                        res.finish_reason = why
                        model.close_sequence(slot_of.pop(r))
                if not ahead:
                    break
                rows, sampled, handle, n_step_tokens = ahead, sampled_ahead, handle_ahead, len(ahead)
                if not any(r in slot_of for r in rows):  # all of them ended at stop tokens meanwhile
                    model.finish_fetch(handle)
                    break
        finally:
            for slot in slot_of.values():
                model.close_sequence(slot)

    def _account(self, prompt_step: bool, n_tokens: int, dt: float, sampling_events) -> None:
        st = self.stats
        if prompt_step:
            st.prefill_steps, st.prefill_tokens, st.prefill_s = st.prefill_steps + 1, st.prefill_tokens + n_tokens, st.prefill_s + dt
        else:
            st.decode_steps, st.decode_tokens, st.decode_s = st.decode_steps + 1, st.decode_tokens + n_tokens, st.decode_s + dt
        if self.stage_timings is not None:
            ms = self.model.stage_times()
            if sampling_events is not None:
                ms["sampling"] = ms.get("sampling", 0.0) + sampling_events[0].elapsed_time(sampling_events[1])
            self.stage_timings["prefill" if prompt_step else "decode"].add(ms, n_tokens)
