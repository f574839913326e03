"""Choosing the next token from float32 logits on the device.

Options and their meanings are the reference's (crates/runner/src/main.rs:370-387;
crates/runner/src/qwen36_moe_decode.rs:1107-1185): ``temperature`` 0 (or ``top_k`` 1)
is greedy argmax with the lowest index winning ties; otherwise logits are scaled by
1/temperature, cut to the ``top_k`` largest (0 = no cut), turned into probabilities,
cut to the smallest set reaching ``top_p`` (1.0 = no cut), and one token is drawn.
Each sequence draws from its own xorshift64 generator kept beside its cache slot,
seeded from ``sampling_seed`` and the request's index, so a sequence's tokens do not
depend on what else is in its batch.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    sampling_seed: int = 42

    def __post_init__(self):
        if self.temperature < 0 or self.top_k < 0 or not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"bad sampling parameters: {self}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


def request_seed(sampling_seed: int, request_index: int) -> int:
    """Generator state for one request: splitmix64 of (seed, index), never zero."""
    z = (int(sampling_seed) + 0x9E3779B97F4A7C15 * (int(request_index) + 1)) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    z ^= z >> 31
    return z or 0x9E3779B97F4A7C15


class Sampler:
    """``__call__(logits [n, vocab] float32, slots [n] int32) -> tokens [n] int32`` on the device."""

    def __init__(self, kernels, rng_state: torch.Tensor):
        self.kernels, self.rng_state = kernels, rng_state

    def __call__(self, logits: torch.Tensor, slots: torch.Tensor, params: SamplingParams) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        if params.greedy:
            self.kernels.argmax(logits, out)
        else:
            self.kernels.sample(logits, params.temperature, params.top_k, params.top_p, slots,
                                self.rng_state, out)
        return out
