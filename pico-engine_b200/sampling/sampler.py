"""Choosing next tokens from logits on the device."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import kernels


@dataclass(frozen=True)
class SamplingParams:
    """Names, defaults and meanings of pico-engine's sampler (src/pico_engine/sampler.py:8-27,
    src/pico_engine/__main__.py:25-28): ``temperature <= 0`` is greedy; ``top_k`` 0 is off and
    keeps ties with the k-th largest; ``top_p`` keeps the smallest set of most likely tokens
    whose mass reaches it (1.0 is off).  ``seed`` names the stream of draws, which the project
    leaves to torch's global generator."""
    temperature: float = 0.7
    top_k: int = 0
    top_p: float = 0.9
    seed: int = 0

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError("top_k must be non-negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must lie in (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0


class Sampler:
    def __init__(self, params: SamplingParams):
        self.params = params

    def kind(self, vocab: int) -> tuple:
        """What fixes the kernels that a choice launches: (greedy, a cut by rank, a cut by mass).  Samplers of
        one kind differ in numbers only (temperature, k, p, seed), which a captured launch reads at run time."""
        p = self.params
        return (True, False, False) if p.greedy else (False, 0 < p.top_k < vocab, p.top_p < 1.0)

    def choose(self, logits: torch.Tensor, request: torch.Tensor, step: torch.Tensor,
               out: torch.Tensor | None = None, settings: torch.Tensor | None = None) -> torch.Tensor:
        """int32 [B] next tokens for float32 logits [B, V].  Row b draws with the uniform of
        (seed, request[b], step[b]); greedy choice ignores both.  ``settings``: int32 [6] on the device
        (``kernels.sample_settings_words``) from which the kernels take temperature, top-k, top-p and seed
        instead of from this sampler's parameters, which then only say which kind of choice it is."""
        p = self.params
        if p.greedy:
            return kernels.argmax(logits, out)
        return kernels.sample(logits, p.temperature, p.top_k, p.top_p, p.seed, request, step, out, settings)
