"""Sampling: greedy, temperature, top-k and top-p."""
from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]
