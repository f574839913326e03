"""Greedy, temperature, top-k and top-p sampling."""
from .sampler import Sampler, SamplingParams, request_seed

__all__ = ["Sampler", "SamplingParams", "request_seed"]
