"""One decode step (every row brings one token) captured as a CUDA graph, for a fixed number of
rows.  All that changes from step to step lives in one int32 device buffer that the host
refreshes before each replay: token ids, positions, page tables, and the sampling counters.

pico-engine captures its one-token forward the same way (src/pico_engine/engine.py:269-306):
static token and position buffers, three warm-up runs on a side stream, replay per token,
eager fallback with a warning if capture fails.
"""
from __future__ import annotations

import warnings
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import pages_for
from .step import StepLayout, Stepper


class GraphedDecode:
    def __init__(self, stepper: Stepper, sampler, B: int):
        self.stepper, self.sampler, self.B = stepper, sampler, B
        cache = stepper.cache
        self.widths = [pages_for(stepper.max_context)] * len(cache.groups)
        self.layout = StepLayout(B, B, B, self.widths)
        n = self.layout.total
        self.extra = n                                   # request ids [B], then step counters [B]
        self.dev = torch.zeros(n + 2 * ((B + 3) & ~3), dtype=torch.int32, device=stepper.device)
        self.host = np.zeros(self.dev.numel(), dtype=np.int32)
        self.tokens_out = torch.zeros(B, dtype=torch.int32, device=stepper.device)
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.failed = False
        self._tables_of: Optional[tuple] = None

    # ------------------------------------------------------------------ host side of a step
    def _fill(self, slots: Sequence[int], tokens: Sequence[int], requests: Sequence[int], steps: Sequence[int]) -> None:
        lay, cache, B = self.layout, self.stepper.cache, self.B
        lens = [1] * B
        _, fresh, starts = self.stepper.describe(slots, lens, None, [[t] for t in tokens], self.widths)
        self.host[:lay.total] = fresh
        pad = (B + 3) & ~3
        self.host[self.extra: self.extra + B] = np.asarray(requests, dtype=np.int32)
        self.host[self.extra + pad: self.extra + pad + B] = np.asarray(steps, dtype=np.int32)
        self._starts, self._slots = starts, list(slots)

    def _forward(self) -> None:
        lay, B = self.layout, self.B
        pad = (B + 3) & ~3
        ctx = self.stepper.context(lay, self.dev, [1] * B, [0] * B, self._slots)
        ctx.max_context = self.stepper.max_context       # launch shapes must not depend on the step
        ctx.starts = [self.stepper.max_context - 1] * B
        ids = self.dev[lay.ids: lay.ids + B]
        self.logits = self.stepper.model.forward(ids, ctx, self.dev[lay.want: lay.want + B])
        self.sampler.choose(self.logits, self.dev[self.extra: self.extra + B],
                            self.dev[self.extra + pad: self.extra + pad + B], self.tokens_out)

    def _capture(self) -> None:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):                           # the step is idempotent: it rewrites the same cache rows
                self._forward()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._forward()
        self.graph = graph

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def run(self, slots: Sequence[int], tokens: Sequence[int], requests: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """One decode step of ``B`` rows; returns the chosen tokens (int32 [B], device)."""
        self._fill(slots, tokens, requests, steps)
        self.stepper.upload(self.host, self.dev)
        if self.graph is None and not self.failed:
            try:
                self._capture()
            except Exception as e:                       # noqa: BLE001 - any capture failure means eager decode
                self.failed = True
                warnings.warn(f"CUDA graph capture failed; decoding without a graph: {e}")
        if self.graph is not None:
            self.graph.replay()
        else:
            self._forward()
        for s in slots:
            self.stepper.cache.advance(s, 1)
        return self.tokens_out
