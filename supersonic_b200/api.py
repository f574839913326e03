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


def load(model_dir: str, dtype: str = "bfloat16", device: int = 0, context_size: Optional[int] = None,
         batch_size: int = 1, max_tokens: Optional[int] = None,
         step_token_budget: Optional[int] = None) -> Engine:
    """Load ``model_dir`` (config.json + safetensors).  The cache holds ``max_tokens`` tokens
    in all, by default ``batch_size`` sequences of ``context_size`` tokens (prompt plus
    generated; default: the model's position limit, capped at 8192).  A step of more than
    ``step_token_budget`` tokens (default 32,768) runs in chunks of that many: it bounds the
    memory a batch of long prompts needs beside the cache."""
    from .cache import PAGE_TOKENS
    from .config import load_config
    cfg = load_config(model_dir)
    ctx = context_size or min(getattr(cfg, "max_position_embeddings", 8192), 8192)
    ctx = -(-ctx // PAGE_TOKENS) * PAGE_TOKENS
    total = max_tokens or ctx * max(batch_size, 1)
    extra = {} if step_token_budget is None else {"step_token_budget": step_token_budget}
    model = Model.from_dir(model_dir, dtype=dtype, device=f"cuda:{device}", max_tokens=total,
                           max_seq_tokens=ctx, **extra)
    return Engine(model)
