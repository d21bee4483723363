"""The Python entry point: a model folder in, generated token ids out.

In pico-engine's manner (src/pico_engine/engine.py:16-24, 308-337): ``Engine(path)`` loads,
``Engine.generate(prompt, max_tokens=64, temperature=0.7, top_k=0, top_p=0.9, use_graph=True)``
generates.  Differences that the scope brings: prompts and results are token ids (there is no
tokenizer here), ``generate`` also takes a batch of prompts, and draws are seeded.
"""
from __future__ import annotations

import os
import time
from typing import Iterable, List, Optional, Sequence, Union

import torch

from ..cache import Cache, PAGE
from ..config.registry import architecture, read_config
from ..ops import kernels
from ..ops.library import core, require_cuda
from ..sampling import Sampler, SamplingParams
from ..weights import load_folder, load_into, random_tensor
from .generate import Request, cut_prompts, generate as run_generation, held_tokens
from .graph import GraphedDecode, TokenLoop, bucket_rows
from .step import Stepper

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(d) -> torch.dtype:
    try:
        return DTYPES[d]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {d!r}") from None


class Engine:
    """A loaded model with its cache, step function and generation loop on one CUDA device.

    ``max_tokens_in_cache``: the most tokens live sequences hold at any time, each rounded up to a
    page of 64; ``max_context``: the longest single sequence; ``max_batch``: sequences per batch;
    ``prefill_tokens_per_step`` (an attribute, 16,384): the most prompt tokens one step takes.
    The cache is allocated on first use and grows when a call needs more.
    """

    def __init__(self, model_path: Union[str, os.PathLike, None], device: str = "cuda", dtype="bfloat16",
                 max_tokens_in_cache: Optional[int] = None, max_context: Optional[int] = None, max_batch: int = 64,
                 _config=None, _seed: Optional[int] = None, _draw_on="cpu"):
        self.device = require_cuda(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.dtype = _dtype(dtype)
        core()                                              # build or load the kernels now, loudly
        torch.cuda.set_device(self.device)
        self.config = _config if _config is not None else read_config(os.fspath(model_path))
        arch = architecture(self.config.ARCHITECTURE)
        self.model = arch.build_model(self.config, self.dtype, self.device)
        if _config is None:
            load_folder(self.model, os.fspath(model_path))
        else:
            expected = self.model.expected_tensors()
            store = torch.bfloat16
            load_into(self.model, lambda n: random_tensor(n, expected[n], _seed, store, _draw_on),
                      {n: s.shape for n, s in expected.items()}, "the random weights")
        self.max_batch = max_batch
        self.prefill_tokens_per_step = 16384      # prompts of a batch beyond this many tokens are run in several steps
        self._want_tokens = max_tokens_in_cache
        self._want_context = max_context
        self.cache: Optional[Cache] = None
        self.stepper: Optional[Stepper] = None
        self._graphs = {}
        self._token_loop: Optional[TokenLoop] = None
        self.last_timing = {}                     # host-clock seconds of the last generate call, by phase

    @classmethod
    def from_config(cls, config, seed: int = 0, draw_on="cpu", **kwargs) -> "Engine":
        """An engine with random weights drawn from ``config`` and ``seed``, without a model
        folder: the values the random-weights writer would store in bfloat16.  ``draw_on`` "cuda"
        draws on the device, which is quicker for large models and gives other values."""
        return cls(None, _config=config, _seed=seed, _draw_on=draw_on, **kwargs)

    # ------------------------------------------------------------------ cache
    def ensure_cache(self, max_tokens: int, max_context: int, max_seqs: Optional[int] = None) -> None:
        """Make the cache hold ``max_tokens`` tokens (in pages) and sequences of ``max_context``."""
        max_tokens = max(max_tokens, self._want_tokens or 0, PAGE)
        max_context = min(max(max_context, self._want_context or 0, 1), self.model.plan.max_positions)
        max_seqs = max_seqs or max(self.max_batch, 1)
        c = self.cache
        if c is not None and c.n_pages * PAGE >= max_tokens and self.stepper.max_context >= max_context \
                and c.max_seqs >= max_seqs:
            return
        if c is not None and c.lengths:
            raise RuntimeError("the cache cannot grow while sequences are open")
        if c is not None:                                   # it only ever grows: what it held it keeps holding
            max_tokens = max(max_tokens, c.n_pages * PAGE)
            max_context = max(max_context, self.stepper.max_context)
            max_seqs = max(max_seqs, c.max_seqs)
        self.cache = self.stepper = None
        self._graphs.clear()
        self.cache = Cache(self.model.cache_needs(), max_tokens, max_seqs, self.dtype, self.device)
        self.model.prepare(max_context)
        self.stepper = Stepper(self.model, self.cache, max_context)

    # ------------------------------------------------------------------ generation
    @torch.inference_mode()
    def generate(self, prompt: Union[Sequence[int], Sequence[Sequence[int]]], max_tokens: Union[int, Sequence[int]] = 64,
                 temperature: float = 0.7, top_k: int = 0, top_p: float = 0.9, use_graph: bool = True,
                 seed: int = 0, stop_token_ids: Optional[Iterable[int]] = None):
        """Generated token ids: a list for one prompt (a list of ints), a list of lists for a
        batch of prompts.  ``stop_token_ids`` defaults to the configuration's eos ids; a stop
        token ends its sequence and is not returned."""
        single = len(prompt) > 0 and isinstance(prompt[0], int) or len(prompt) == 0
        prompts = [list(prompt)] if single else [list(p) for p in prompt]
        requests = self.generate_requests(prompts, max_tokens, SamplingParams(temperature, top_k, top_p, seed),
                                          use_graph, stop_token_ids)
        outs = [r.output for r in requests]
        return outs[0] if single else outs

    def generate_requests(self, prompts, max_tokens, params: SamplingParams, use_graph: bool = True,
                          stop_token_ids: Optional[Iterable[int]] = None) -> List[Request]:
        stop = tuple(self.model.plan.stop_token_ids) if stop_token_ids is None else tuple(stop_token_ids)
        mnt = [max_tokens] * len(prompts) if isinstance(max_tokens, int) else list(max_tokens)
        probe = [Request(i, list(p), m) for i, (p, m) in enumerate(zip(prompts, mnt)) if len(p)]
        if probe:
            need = [held_tokens(r) for r in probe]
            budget = self._want_tokens or sum(sorted(need, reverse=True)[:self.max_batch])
            self.ensure_cache(max(budget, max(need)), max(len(r.prompt) + max(r.max_new_tokens - 1, 0) for r in probe))
        self.last_timing = {"prefill_s": 0.0, "decode_s": 0.0, "decode_steps": 0, "h2d_bytes": 0}
        backend = EngineBackend(self, Sampler(params), use_graph)
        budget = self.cache.n_pages * PAGE if self.cache is not None else PAGE
        requests = run_generation(backend, prompts, mnt, stop, self.max_batch, budget)
        kernels.check_status(self.device)
        return requests


class EngineBackend:
    """The generation loop's backend on the engine's stepper: steps, then chooses on the device
    and hands the chosen tokens to the host."""

    def __init__(self, engine: Engine, sampler: Sampler, use_graph: bool):
        self.e, self.sampler, self.use_graph = engine, sampler, use_graph
        self._mark = None                                # when the decode time counted so far ends

    def open(self) -> int:
        return self.e.cache.open()

    def close(self, slot: int) -> None:
        self.e.cache.close(slot)

    def _int32(self, values) -> torch.Tensor:
        return torch.tensor(list(values), dtype=torch.int32).to(self.e.device, non_blocking=True)

    def prefill(self, slots, prompts, requests) -> List[int]:
        """The prompts of a batch: in one step, or, where they have more tokens than ``Engine.prefill_tokens_per_step``,
        in several (the activations of a step grow with its tokens: the cache may hold a batch whose prompts in one
        step would not fit beside it).  A prompt's later pieces start inside its sequence; the logits that choose a
        request's first token are those of its last piece's last token."""
        t0 = time.perf_counter()
        budget = self.e.prefill_tokens_per_step
        if sum(len(p) for p in prompts) <= budget:
            logits = self.e.stepper.step(slots, prompts, use_graph=self.use_graph)
        else:
            rows = [None] * len(slots)
            for pieces in cut_prompts([len(p) for p in prompts], budget):
                ends = [at + n == len(prompts[r]) for r, at, n in pieces]
                out = self.e.stepper.step([slots[r] for r, _, _ in pieces], [prompts[r][at:at + n] for r, at, n in pieces],
                                          [[n - 1] if end else [] for (_, _, n), end in zip(pieces, ends)])
                for k, r in enumerate(r for (r, _, _), end in zip(pieces, ends) if end):
                    rows[r] = out[k]
            logits = torch.stack(rows)
        chosen = self.sampler.choose(logits, self._int32(requests), self._int32([0] * len(slots))).tolist()
        self.e.last_timing["prefill_s"] += time.perf_counter() - t0
        return chosen

    MAX_GRAPHS = 24      # captured decode steps an engine keeps (each holds its buffers); the least recently used goes

    def _graph(self, rows: int) -> GraphedDecode:
        """The captured step for ``rows`` rows: one per bucket of rows and kind of sampling.  Temperature,
        top-k, top-p and seed are numbers the graph reads at run time, so calls that vary them share it."""
        key = (bucket_rows(rows), self.sampler.kind(self.e.model.plan.vocab_size))
        graphs = self.e._graphs
        g = graphs.pop(key, None)
        if g is None:
            if self.e._token_loop is None:
                self.e._token_loop = TokenLoop(self.e.device)
            g = GraphedDecode(self.e.stepper, self.sampler, key[0], self.e._token_loop)
            while len(graphs) >= self.MAX_GRAPHS:
                graphs.pop(next(iter(graphs)))
        graphs[key] = g                                  # most recently used last
        return g

    def decode(self, slots, tokens, requests, steps) -> List[int]:
        """One token per sequence in, one chosen token per sequence out, both on the host: the
        step's description is copied from pinned memory, the result is read back."""
        t0, sent = time.perf_counter(), self.e.stepper.h2d_bytes
        if self.use_graph:
            chosen = self._graph(len(slots)).launch(slots, tokens, requests, steps, sampler=self.sampler).tokens()
        else:
            logits = self.e.stepper.step(slots, [[t] for t in tokens])
            chosen = self.sampler.choose(logits, self._int32(requests), self._int32(steps)).tolist()
        t = self.e.last_timing
        t["decode_s"] += time.perf_counter() - t0
        t["decode_steps"] += 1
        t["h2d_bytes"] += self.e.stepper.h2d_bytes - sent
        return chosen

    # The same step in two halves, so that the loop can launch the next step before it reads this
    # one's tokens (only with graphs: the next step then takes its ids on the device).
    @property
    def pipelined(self) -> bool:
        return self.use_graph

    def decode_begin(self, slots, tokens, sources, requests, steps):
        """Launch a decode step.  ``sources[j] >= 0`` names the row of the step launched just before
        whose chosen token is row j's input (``tokens[j]`` is then ignored)."""
        now, sent = time.perf_counter(), self.e.stepper.h2d_bytes
        if self._mark is None:
            self._mark = now
        flight = self._graph(len(slots)).launch(slots, [0 if s >= 0 else t for t, s in zip(tokens, sources)],
                                                requests, steps, sources, sampler=self.sampler)
        t = self.e.last_timing
        t["decode_steps"] += 1
        t["h2d_bytes"] += self.e.stepper.h2d_bytes - sent
        return flight

    def decode_end(self, flight) -> List[int]:
        chosen = flight.tokens()
        now = time.perf_counter()
        self.e.last_timing["decode_s"] += now - self._mark      # wall time since the last step ended (or the first began)
        self._mark = now
        return chosen

    def decode_idle(self) -> None:
        """No step is in flight any more: the time until the next one begins is not decoding."""
        self._mark = None
