"""One decode step (every row brings one token) captured as a CUDA graph, for a fixed number of
rows.  All that changes from step to step lives in one int32 device buffer that the host
refreshes before each replay: token ids, positions, page tables, the sampling counters and the
sampler's settings (temperature, top-k, top-p, seed).  A graph is captured for a *bucket* of rows
(1, 2, 4, 8, ...): a step of fewer rows fills the bucket with idle rows, which bring token 0 at
position 0 of the cache's idle slot and whose results nobody reads, so that a batch whose requests
end one by one needs a handful of graphs, not one per row count.  A step may also take its token
ids from what the step before it chose, on the device, so that the host can launch it before it
has read those tokens (``TokenLoop``).

pico-engine captures its one-token forward the same way (src/pico_engine/engine.py:269-306):
static token and position buffers, three warm-up runs on a side stream, replay per token,
eager fallback with a warning if capture fails.
"""
from __future__ import annotations

import gc
import warnings
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import pages_for
from ..ops import kernels
from .step import StepLayout, Stepper


class InFlight:
    """A decode step that has been launched: its chosen tokens are on their way to pinned host memory."""

    def __init__(self, B: int, staged: torch.Tensor, done: "torch.cuda.Event"):
        self.B, self.staged, self.done = B, staged, done

    def tokens(self) -> List[int]:
        """Wait for the step and return its chosen tokens."""
        self.done.synchronize()
        return self.staged[:self.B].tolist()


class TokenLoop:
    """What the decode graphs of one engine share so that a step can follow another without the
    host in between: the device buffer into which every step writes its chosen tokens (the next
    step takes its token ids from there) and pinned host buffers for reading them back."""

    ROWS = 4096

    def __init__(self, device):
        self.chosen = torch.zeros(self.ROWS, dtype=torch.int32, device=device)
        self._pinned = [torch.zeros(self.ROWS, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._events = [torch.cuda.Event() for _ in range(4)]
        self._at = 0

    def read_back(self, B: int) -> InFlight:
        """Copy the tokens the last step chose to the host, in stream order, without waiting."""
        i = self._at
        self._at = (i + 1) % len(self._pinned)
        self._pinned[i][:B].copy_(self.chosen[:B], non_blocking=True)
        self._events[i].record()
        return InFlight(B, self._pinned[i], self._events[i])


class _collector_paused:
    """While a capture records, Python's cycle collector stays off: were it to free an object that owns a captured graph
    or other device resources in the middle of the capture, the release would be a forbidden operation on a capturing
    stream and break the capture.  (torch's capture context collects once before it starts.)"""

    def __enter__(self):
        self.was_on = gc.isenabled()
        gc.disable()

    def __exit__(self, *exc):
        if self.was_on:
            gc.enable()


def _leave_failed_capture(stream) -> None:
    """After a capture that raised: torch's capture context has not put the stream back that was current before it
    (its exit stops at the failed end of the capture), so work launched next would go to the stream whose capture
    broke and fail with it.  Make ``stream`` current again and let the device drain."""
    torch.cuda.set_stream(stream)
    try:
        torch.cuda.synchronize()
    except Exception:                                     # noqa: BLE001 - the error of the capture, reported once more
        pass


PROMPT_TOKEN_STEP = 128       # a captured prompt step holds a multiple of this many tokens
PROMPT_IDLE_ROWS = 2          # and at least this many idle rows, which take up to a page of padding tokens each


def prompt_sizes(n_rows: int, n_tokens: int) -> tuple:
    """(rows, tokens) of the captured step that runs ``n_rows`` prompts of ``n_tokens`` tokens together: the rows of
    the next power of two and two more, the tokens of the next multiple of 128.  (An idle row brings between no token
    and a page of 64: two of them take any padding up to 127 tokens.)"""
    rows = bucket_rows(n_rows) + PROMPT_IDLE_ROWS
    tokens = (n_tokens + PROMPT_TOKEN_STEP - 1) // PROMPT_TOKEN_STEP * PROMPT_TOKEN_STEP
    return rows, tokens


class GraphedPrompt:
    """A step whose rows bring their prompts (or pieces of them), captured as a CUDA graph for fixed sizes: ``T`` packed
    tokens, ``B`` rows, a fixed number of attention runs, the widest page tables.  A step of fewer rows and tokens fills
    up with idle rows: tokens 0 at the first positions of the cache's idle slot, whose results nobody reads.  Replayed,
    the step costs the host one description and one copy instead of a launch per kernel (for a 2,048-token prompt of
    the Qwen2.5-0.5B shape 2.6 ms instead of 3.1, for 512 tokens 1.5 ms instead of 2.9).  The first step of some sizes
    runs kernel by kernel at the same padded sizes, the second is captured: the kernels and their results are the same
    either way, so a call's tokens do not depend on whether its sizes have been seen before."""

    def __init__(self, stepper: Stepper, B: int, T: int, pool=None):
        self.stepper, self.B, self.T, self.pool = stepper, B, T, pool
        self.widths = [pages_for(stepper.max_context)] * len(stepper.cache.groups)
        self.n_tiles = (T // kernels.PREFILL_TILE + B, T // kernels.PREFILL_TILE_TCGEN05 + B)
        self.layout = StepLayout(T, B, B, self.widths, self.n_tiles)
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=stepper.device)
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.failed = False
        self.launches = 0                                 # the first runs kernel by kernel, the second captures

    @staticmethod
    def padding(n_rows: int, n_tokens: int, B: int, T: int) -> List[int]:
        """Tokens of each of the ``B - n_rows`` idle rows so that the step has ``T`` tokens: a page of 64 at most."""
        idle, pad = B - n_rows, T - n_tokens
        if idle < 0 or not 0 <= pad <= idle * 64:
            raise ValueError(f"{n_rows} rows of {n_tokens} tokens do not fit a captured step of {B} rows and {T} tokens")
        out = []
        for _ in range(idle):
            out.append(min(64, pad))
            pad -= out[-1]
        return out

    def _forward(self, ctx) -> None:
        lay = self.layout
        self.logits = self.stepper.model.forward(self.dev[lay.ids: lay.ids + lay.T], ctx, self.dev[lay.want: lay.want + lay.W])

    @torch.inference_mode()
    def launch(self, slots: Sequence[int], token_ids: Sequence[Sequence[int]]) -> torch.Tensor:
        """Run the rows' tokens; returns float32 logits [len(slots), vocab] at each row's last token."""
        st, cache, lay = self.stepper, self.stepper.cache, self.layout
        lens = [len(t) for t in token_ids]
        pad = self.padding(len(slots), sum(lens), self.B, self.T)
        all_slots = list(slots) + [cache.idle_slot] * len(pad)
        _, host, starts = st.describe(all_slots, lens + pad, None, list(token_ids) + [[0] * n for n in pad], self.widths, self.n_tiles)
        st.upload(host, self.dev)
        ctx = st.context(lay, self.dev, lens + pad, starts, all_slots)
        ctx.max_context = st.max_context                  # what the captured launches were shaped for
        self.launches += 1
        if self.graph is None and not self.failed and self.launches >= 2:
            stream = torch.cuda.current_stream()
            try:
                state = cache.snapshot_state()            # the trial runs must not advance a mixer's state (see GraphedDecode)
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._forward(ctx)                    # (the step ran kernel by kernel before: everything lazy is set up)
                    cache.restore_state(state)
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with _collector_paused(), torch.cuda.graph(graph, pool=self.pool):
                    self._forward(ctx)
                self.graph = graph
            except Exception as e:                        # noqa: BLE001 - any capture failure means launching kernel by kernel
                self.failed = True
                _leave_failed_capture(stream)
                warnings.warn(f"CUDA graph capture of a prompt step failed; it runs without a graph: {e}")
        if self.graph is not None:
            self.graph.replay()
        else:
            self._forward(ctx)
        for s, n in zip(slots, lens):
            cache.advance(s, n)
        return self.logits[:len(slots)]


def bucket_rows(rows: int) -> int:
    """The number of rows of the graph that runs a decode step of ``rows`` rows: the next power of two."""
    b = 1
    while b < rows:
        b *= 2
    return b


class GraphedDecode:
    """``B`` is the number of rows of the captured step; a launch may bring fewer.  ``sampler`` says how tokens
    are chosen (greedy, or which cuts a draw makes: that fixes the kernels of the graph); its temperature,
    top-k, top-p and seed are read from the device buffer at run time, so one graph serves every setting
    of the same kind (``launch(..., sampler=)``)."""

    def __init__(self, stepper: Stepper, sampler, B: int, loop: Optional[TokenLoop] = None):
        self.stepper, self.sampler, self.B = stepper, sampler, B
        cache = stepper.cache
        self.loop = loop or TokenLoop(stepper.device)
        if B > TokenLoop.ROWS:
            raise ValueError(f"a decode step of {B} rows is more than the {TokenLoop.ROWS} the token buffer holds")
        self.widths = [pages_for(stepper.max_context)] * len(cache.groups)
        self.layout = StepLayout(B, B, B, self.widths)
        n = self.layout.total
        self.extra = n                                   # request ids [B], step counters [B], token sources [B], settings [6]
        self.pad = (B + 3) & ~3
        self.settings_at = n + 3 * self.pad              # a multiple of 4 words: the 64-bit seed is aligned
        self.dev = torch.zeros(self.settings_at + 8, dtype=torch.int32, device=stepper.device)
        self.host = np.zeros(self.dev.numel(), dtype=np.int32)
        self.tokens_out = self.loop.chosen[:B]
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.failed = False
        self._tables_of: Optional[tuple] = None

    # ------------------------------------------------------------------ host side of a step
    def _fill(self, slots: Sequence[int], tokens: Sequence[int], requests: Sequence[int], steps: Sequence[int],
              sources: Optional[Sequence[int]], sampler) -> None:
        lay, B, pad, n = self.layout, self.B, self.pad, len(slots)
        if n > B:
            raise ValueError(f"a step of {n} rows does not fit a graph of {B}")
        idle = [self.stepper.cache.idle_slot] * (B - n)
        _, fresh, starts = self.stepper.describe(list(slots) + idle, [1] * B, None, [[t] for t in tokens] + [[0]] * (B - n),
                                                 self.widths)
        self.host[:lay.total] = fresh
        self.host[self.extra: self.extra + B] = 0
        self.host[self.extra: self.extra + n] = np.asarray(requests, dtype=np.int32)
        self.host[self.extra + pad: self.extra + pad + B] = 0
        self.host[self.extra + pad: self.extra + pad + n] = np.asarray(steps, dtype=np.int32)
        self.host[self.extra + 2 * pad: self.extra + 2 * pad + B] = -1
        if sources is not None:
            self.host[self.extra + 2 * pad: self.extra + 2 * pad + n] = np.asarray(sources, dtype=np.int32)
        p = (sampler or self.sampler).params
        if (sampler or self.sampler).kind(self.stepper.vocab) != self.sampler.kind(self.stepper.vocab):
            raise ValueError("this graph was captured for another kind of sampling")
        self.host[self.settings_at: self.settings_at + 6] = kernels.sample_settings_words(
            p.temperature if p.temperature > 0 else 1.0, p.top_k, p.top_p, p.seed)
        self._starts, self._slots = starts, list(slots) + idle

    def _forward(self) -> None:
        lay, B, pad = self.layout, self.B, self.pad
        ctx = self.stepper.context(lay, self.dev, [1] * B, [0] * B, self._slots)
        ctx.max_context = self.stepper.max_context       # launch shapes must not depend on the step
        ctx.starts = [self.stepper.max_context - 1] * B
        ids = self.dev[lay.ids: lay.ids + B]
        # rows whose token the host has not seen take it from the step before, on the device
        kernels.select_tokens(ids, self.loop.chosen, self.dev[self.extra + 2 * pad: self.extra + 2 * pad + B])
        self.logits = self.stepper.model.forward(ids, ctx, self.dev[lay.want: lay.want + B])
        self.sampler.choose(self.logits, self.dev[self.extra: self.extra + B],
                            self.dev[self.extra + pad: self.extra + pad + B], self.tokens_out,
                            settings=self.dev[self.settings_at: self.settings_at + 6])

    def _capture(self) -> None:
        # The warm-up runs and the capture write the shared token buffer; what the step before chose
        # is kept aside meanwhile, since this step may take its ids from there.  Keys and values are
        # rewritten with the same numbers by every run, but per-sequence state (a mixer's running sums) would
        # be advanced once per run: it is put back after the warm-up, so that only the replay counts.
        keep = self.loop.chosen.clone()
        state = self.stepper.cache.snapshot_state()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.loop.chosen.copy_(keep)
                self._forward()
            self.stepper.cache.restore_state(state)
        torch.cuda.current_stream().wait_stream(side)
        self.loop.chosen.copy_(keep)
        graph = torch.cuda.CUDAGraph()
        with _collector_paused(), torch.cuda.graph(graph):
            self._forward()
        self.loop.chosen.copy_(keep)
        self.graph = graph

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def launch(self, slots: Sequence[int], tokens: Sequence[int], requests: Sequence[int], steps: Sequence[int],
               sources: Optional[Sequence[int]] = None, sampler=None) -> InFlight:
        """Start one decode step of ``len(slots) <= B`` rows and the copy of its chosen tokens to the host.
        Row j's token is ``tokens[j]``, or, where ``sources[j] >= 0``, what row ``sources[j]`` of the step
        launched before this one chose (``tokens[j]`` is then any valid id).  ``sampler``: the settings of
        this step's draws (of the kind the graph was captured for); default: the sampler of the capture."""
        self._fill(slots, tokens, requests, steps, sources, sampler)
        self.stepper.upload(self.host, self.dev)
        if self.graph is None and not self.failed:
            stream = torch.cuda.current_stream()
            try:
                self._capture()
            except Exception as e:                       # noqa: BLE001 - any capture failure means eager decode
                self.failed = True
                _leave_failed_capture(stream)
                warnings.warn(f"CUDA graph capture failed; decoding without a graph: {e}")
        if self.graph is not None:
            self.graph.replay()
        else:
            self._forward()
        for s in slots:
            self.stepper.cache.advance(s, 1)
        return self.loop.read_back(len(slots))

    def run(self, slots: Sequence[int], tokens: Sequence[int], requests: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """One decode step; returns the chosen tokens (int32 [B], device; the first ``len(slots)`` count)."""
        self.launch(slots, tokens, requests, steps)
        return self.tokens_out
