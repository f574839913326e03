"""The Python entry point: load a model folder, generate token ids.

The reference has no Python API (its Python files are oracle and bake tooling); the
options here carry the names and meanings of its command line
(crates/runner/src/main.rs:347-402, 646): ``max_new_tokens`` (8), ``temperature`` (0 =
greedy), ``top_k`` (0 = off), ``top_p`` (1.0 = off), ``sampling_seed`` (42),
``context_size``, ``device``, ``batch_size``.  Token ids in, token ids out.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

from .engine.generate import GenerationResult, Generator
from .engine.model import Model
from .sampling import SamplingParams


class Engine:
    """A loaded model with its cache and generation loop."""

    def __init__(self, model: Model):
        self.model = model
        self.generator = Generator(model)

    @property
    def config(self):
        return self.model.config

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 8,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 sampling_seed: int = 42, stop_token_ids: Optional[Sequence[int]] = None,
                 ignore_eos: bool = False, include_stop_token: bool = True,
                 batch_size: Optional[int] = None) -> List[List[int]]:
        """Generated token ids for each prompt (a list of token-id lists)."""
        return [r.tokens for r in self.generate_detailed(
            prompts, max_new_tokens, temperature, top_k, top_p, sampling_seed, stop_token_ids,
            ignore_eos, include_stop_token, batch_size)]

    def generate_detailed(self, prompts, max_new_tokens=8, temperature=0.0, top_k=0, top_p=1.0,
                          sampling_seed=42, stop_token_ids=None, ignore_eos=False,
                          include_stop_token=True, batch_size=None) -> List[GenerationResult]:
        params = SamplingParams(temperature, top_k, top_p, sampling_seed)
        return self.generator.generate(prompts, max_new_tokens, params, stop_token_ids, ignore_eos,
                                       include_stop_token, batch_size)


    def score(self, sequences: Sequence[Sequence[int]], decode_step: bool = False):
        """Teacher-forced scoring of given token sequences (``engine/score.py``): a list of
        :class:`Score` with total and mean negative log-likelihood, perplexity, bits per token."""
        from .engine.score import teacher_forced
        return teacher_forced(self.model, sequences, decode_step)


def load(model_dir: Optional[str] = None, dtype: str = "bfloat16", device: int = 0,
         context_size: Optional[int] = None, batch_size: int = 1, max_tokens: Optional[int] = None,
         step_token_budget: Optional[int] = None, preset: Optional[str] = None, random_seed: int = 0,
         allow_unexpected_tensors: bool = False, use_graphs: bool = True,
         deterministic: bool = False) -> Engine:
    """Load ``model_dir`` (config.json + safetensors), or build the named ``preset`` with random
    weights made on the device from ``random_seed`` (no folder is read or written).  The cache holds
    ``max_tokens`` tokens in all, by default ``batch_size`` sequences of ``context_size`` tokens
    (prompt plus generated; default: the model's position limit, capped at 8192).  A step of more
    than ``step_token_budget`` tokens (default 32,768) runs in chunks of that many: it bounds the
    memory a batch of long prompts needs beside the cache.  Weights, cache and workspace are checked
    against the device's free memory before anything is loaded.  ``deterministic``: the bfloat16
    path without float atomics, so that the same batch gives the same bits every run and sampled
    tokens are reproducible from their seed (the float32 path always is)."""
    from .cache import PAGE_TOKENS
    from .config import load_config, preset_config
    if (model_dir is None) == (preset is None):
        raise ValueError("give either a model folder or a preset name")
    cfg = load_config(model_dir) if model_dir is not None else preset_config(preset)
    ctx = context_size or min(getattr(cfg, "max_position_embeddings", 8192), 8192)
    ctx = -(-ctx // PAGE_TOKENS) * PAGE_TOKENS
    total = max_tokens or ctx * max(batch_size, 1)
    extra = {"use_graphs": use_graphs, "deterministic": deterministic}
    if step_token_budget is not None:
        extra["step_token_budget"] = step_token_budget
    dev = f"cuda:{device}"
    if model_dir is not None:
        model = Model.from_dir(model_dir, dtype=dtype, device=dev, max_tokens=total, max_seq_tokens=ctx,
                               allow_unexpected_tensors=allow_unexpected_tensors, **extra)
    else:
        from .weights import RandomWeightStore
        # norm weights exactly 1, matrices N(0, 0.02): the sizes-only models of a benchmark
        store = RandomWeightStore(cfg, random_seed, device=dev, std=0.02, norm_jitter=0.0)
        model = Model.from_config(cfg, store, dtype=dtype, device=dev, max_tokens=total, max_seq_tokens=ctx, **extra)
    return Engine(model)
