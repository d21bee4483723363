"""The step function: run the given tokens of a batch of sequences, from the cache, as one
batch, and return the logits at the wanted places.

A step takes sequences that are open in the cache and, for each, the next tokens of that
sequence (a whole prompt, a piece of one, or one decoded token).  Tokens are packed without
padding; the cache is read for everything before them.  After the step the sequences are
longer by what they were given.  pico-engine's counterpart is ``Transformer.forward`` for one
sequence (src/pico_engine/model.py:129-165), whose prompt must start at position 0
(model.py:194-197) and which returns the last row only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import PAGE, Cache, pages_for
from ..ops import kernels
from ..parts.base import StepContext


class StepError(ValueError):
    """A step that cannot run: an empty row, a token outside the vocabulary, a sequence that
    would outgrow the longest one the engine was set up for, a wanted place that is no token
    of this step."""


def _pad4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class StepLayout:
    """Where each array of a step lies in the one int32 buffer that is sent to the device."""
    T: int
    B: int
    W: int
    widths: List[int]
    n_tiles: tuple = (0, 0)          # attention runs of at most 64 and of at most 128 tokens (0, 0: every row brings one token)
    ids: int = 0
    pos: int = 0
    row: int = 0
    slots: int = 0
    first: int = 0
    lens: int = 0
    want: int = 0
    tiles: Optional[List[int]] = None
    tables: Optional[List[int]] = None
    total: int = 0

    def __post_init__(self):
        o = 0
        self.ids = o; o += _pad4(self.T)
        self.pos = o; o += _pad4(self.T)
        self.row = o; o += _pad4(self.T)
        self.slots = o; o += _pad4(self.B)
        self.first = o; o += _pad4(self.B + 1)
        self.lens = o; o += _pad4(self.B)
        self.want = o; o += _pad4(max(self.W, 1))
        self.tiles = []
        for n in self.n_tiles:
            self.tiles.append(o); o += 4 * n
        self.tables = []
        for w in self.widths:
            self.tables.append(o); o += _pad4(self.B * w)
        self.total = o


class Stepper:
    """Owns nothing but scratch: it drives ``model`` over ``cache``."""

    def __init__(self, model, cache: Cache, max_context: int):
        self.model, self.cache, self.max_context = model, cache, max_context
        self.device = cache.device
        self.vocab = model.plan.vocab_size
        self._ring: List[list] = [[None, None] for _ in range(4)]     # pinned staging buffers and their copy events
        self._ring_at = 0
        self.h2d_bytes = 0                        # bytes of step descriptions copied to the device so far
        self._prompt_graphs: dict = {}            # (rows, tokens) -> GraphedPrompt, the most recently used last
        self._prompt_pool = None

    # ------------------------------------------------------------------ building a step
    def _stage(self, host: np.ndarray):
        """A pinned buffer holding ``host``.  Buffers are used in turn; one is written again only
        after the copy that last read it has finished."""
        slot = self._ring[self._ring_at]
        self._ring_at = (self._ring_at + 1) % len(self._ring)
        if slot[1] is not None:
            slot[1].synchronize()
        n = host.shape[0]
        if slot[0] is None or slot[0].numel() < n:
            slot[0] = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        slot[0].numpy()[:n] = host
        return slot, slot[0][:n]

    def describe(self, slots: Sequence[int], lens: Sequence[int], want: Optional[Sequence[Sequence[int]]],
                 token_ids: Optional[Sequence[Sequence[int]]], widths: Optional[List[int]] = None,
                 n_tiles: Optional[tuple] = None):
        """Check the step, reserve its pages and lay its arrays out on the host.

        Returns ``(layout, host int32 array, starts)``.  ``want[b]`` are places among row b's
        tokens of this step; None asks for each row's last token.  ``n_tiles``: how many attention runs
        (of at most 64 and at most 128 tokens) the layout holds, for a step of fixed sizes; where the
        rows make fewer, the last row's first token is listed again (the same result written twice).
        """
        cache = self.cache
        B = len(slots)
        if B == 0:
            raise StepError("a step needs at least one sequence")
        live = [s for s in slots if s != cache.idle_slot]        # idle rows (padding of a fixed-size step) may repeat
        if len(set(live)) != len(live):
            raise StepError("a sequence appears twice in one step")
        lens = [int(n) for n in lens]
        starts = [cache.length(s) for s in slots]
        for b, n in enumerate(lens):
            if slots[b] == cache.idle_slot:
                if not 0 <= n <= PAGE:
                    raise StepError(f"row {b} is idle and brings {n} tokens; the idle slot holds one page of {PAGE}")
                continue
            if n < 1:
                raise StepError(f"row {b} brings no token")
            if starts[b] + n > self.max_context:
                raise StepError(f"row {b} would reach {starts[b] + n} tokens; the engine was set up for sequences "
                                f"of at most {self.max_context}")
        if want is None:
            want = [[n - 1] if n else [] for n in lens]
            empty_rows = sum(1 for n in lens if n == 0)      # idle rows without a token still have a row of logits: of token 0
        else:
            empty_rows = 0
        T = sum(lens)
        W = sum(len(w) for w in want) + empty_rows
        for s, n in zip(live, (n for s, n in zip(slots, lens) if s != cache.idle_slot)):
            cache.reserve(s, n)
        if widths is None:
            widths = [max(pages_for(st + n) for st, n in zip(starts, lens))] * len(cache.groups)
        tile_rows = ([], [])
        if any(n != 1 for n in lens):                    # rows that bring several tokens: the runs the attention kernels take
            tile_rows = tuple(kernels.prefill_tile_rows(lens, starts, t) for t in (kernels.PREFILL_TILE, kernels.PREFILL_TILE_TCGEN05))
            if n_tiles is not None:
                b0 = min((b for b in range(B) if lens[b]), key=lambda b: starts[b])       # the row that starts earliest:
                filler = (b0, sum(lens[:b0]), 1, starts[b0])                                # its first token alone is the cheapest run
                for rows, n in zip(tile_rows, n_tiles):
                    if len(rows) > n:
                        raise StepError(f"the step has {len(rows)} attention runs, its layout holds {n}")
                    rows.extend([filler] * (n - len(rows)))
        lay = StepLayout(T, B, W, widths, tuple(len(r) for r in tile_rows))
        host = np.zeros(lay.total, dtype=np.int32)
        for off, rows in zip(lay.tiles, tile_rows):
            if rows:
                host[off: off + 4 * len(rows)] = np.asarray(rows, dtype=np.int32).reshape(-1)
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        for b in range(B):
            a, e = cu[b], cu[b + 1]
            host[lay.pos + a: lay.pos + e] = np.arange(starts[b], starts[b] + lens[b], dtype=np.int32)
            host[lay.row + a: lay.row + e] = b
            if token_ids is not None:
                ids = np.asarray(token_ids[b], dtype=np.int64)
                if ids.shape != (lens[b],):
                    raise StepError(f"row {b}: {ids.shape[0] if ids.ndim == 1 else ids.shape} tokens given, {lens[b]} announced")
                if ids.size and (ids.min() < 0 or ids.max() >= self.vocab):
                    raise StepError(f"row {b} has a token outside the vocabulary of {self.vocab}")
                host[lay.ids + a: lay.ids + e] = ids
        host[lay.slots: lay.slots + B] = np.asarray(slots, dtype=np.int32)
        host[lay.first: lay.first + B + 1] = cu
        host[lay.lens: lay.lens + B] = np.asarray(lens, dtype=np.int32)
        w_at = lay.want
        for b, places in enumerate(want):
            for p in places:
                if not 0 <= p < lens[b]:
                    raise StepError(f"row {b}: wanted place {p} is none of its {lens[b]} tokens")
                host[w_at] = cu[b] + p
                w_at += 1
        for g, off in enumerate(lay.tables):
            host[off: off + B * widths[g]] = cache.page_table(g, slots, widths[g]).reshape(-1)
        return lay, host, starts

    def context(self, lay: StepLayout, dev: torch.Tensor, lens: List[int], starts: List[int],
                slot_ids: Sequence[int] = ()) -> StepContext:
        tables = {g: dev[off: off + lay.B * lay.widths[g]].view(lay.B, lay.widths[g])
                  for g, off in enumerate(lay.tables)}
        scratch = {name: dev[off: off + 4 * n].view(n, 4)
                   for name, off, n in zip(("prefill_tiles", "prefill_tiles_128"), lay.tiles, lay.n_tiles) if n}
        return StepContext(scratch=scratch,
            T=lay.T, B=lay.B, dtype=self.model.dtype, device=self.device,
            tok_pos=dev[lay.pos: lay.pos + lay.T], tok_row=dev[lay.row: lay.row + lay.T],
            slots=dev[lay.slots: lay.slots + lay.B], row_first=dev[lay.first: lay.first + lay.B + 1],
            row_lens=dev[lay.lens: lay.lens + lay.B], slot_ids=list(slot_ids), lens=list(lens), starts=list(starts),
            one_token_each=all(n == 1 for n in lens), cache=self.cache, tables=tables,
            max_context=max(s + n for s, n in zip(starts, lens)))

    def upload(self, host: np.ndarray, dev: Optional[torch.Tensor] = None) -> torch.Tensor:
        slot, staged = self._stage(host)
        self.h2d_bytes += int(host.nbytes)
        if dev is None:
            dev = torch.empty(host.shape[0], dtype=torch.int32, device=self.device)
        dev[:host.shape[0]].copy_(staged, non_blocking=True)
        if self.device.type == "cuda":
            slot[1] = slot[1] or torch.cuda.Event()
            slot[1].record()
        return dev

    # ------------------------------------------------------------------ the step
    MAX_PROMPT_GRAPHS = 8             # padded prompt steps a stepper keeps (captured ones share one memory pool)
    MAX_GRAPHED_PROMPT_TOKENS = 16384

    def _prompt_graph(self, n_rows: int, n_tokens: int):
        """The padded step that takes ``n_rows`` prompts of ``n_tokens`` tokens.  It is captured as a graph once
        steps of its sizes have come twice (a capture costs two more runs of the step; sizes that never come back
        are not worth one); until then it runs kernel by kernel, at the same padded sizes and so with the same
        kernels and results as the replays that follow."""
        from .graph import GraphedPrompt, prompt_sizes
        key = prompt_sizes(n_rows, n_tokens)
        if key[1] > self.MAX_GRAPHED_PROMPT_TOKENS or self.device.type != "cuda":
            return None
        g = self._prompt_graphs.pop(key, None)
        if g is None:
            if self._prompt_pool is None:
                self._prompt_pool = torch.cuda.graph_pool_handle()
            g = GraphedPrompt(self, key[0], key[1], self._prompt_pool)
            while len(self._prompt_graphs) >= self.MAX_PROMPT_GRAPHS:
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
        self._prompt_graphs[key] = g
        return g

    @torch.inference_mode()
    def step(self, slots: Sequence[int], token_ids: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None,
             device_tokens: Optional[torch.Tensor] = None, use_graph: bool = False) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted places, vocab] on the device, in the
        order of the rows and of ``want``.  With ``device_tokens`` (int32 [B], one token per row,
        already on the device) ``token_ids`` only gives the rows' lengths (all 1).  ``use_graph``: a step
        that brings prompts and wants each row's last logits runs at padded sizes (``engine.graph.GraphedPrompt``:
        rows and tokens filled up with idle rows), from the second time on as a captured graph."""
        if use_graph and want is None and device_tokens is None and any(len(t) != 1 for t in token_ids):
            g = self._prompt_graph(len(slots), sum(len(t) for t in token_ids))
            if g is not None:
                return g.launch(slots, token_ids)
        if device_tokens is not None:
            lens = [1] * len(slots)
            lay, host, starts = self.describe(slots, lens, want, None)
        else:
            lens = [len(t) for t in token_ids]
            lay, host, starts = self.describe(slots, lens, want, token_ids)
        dev = self.upload(host)
        ctx = self.context(lay, dev, lens, starts, slots)
        ids = device_tokens if device_tokens is not None else dev[lay.ids: lay.ids + lay.T]
        x = self.model.hidden(ids, ctx)
        for s, n in zip(slots, lens):
            self.cache.advance(s, n)
        if lay.W == 0:
            return torch.empty(0, self.vocab, dtype=torch.float32, device=self.device)
        return self.model.logits(x, dev[lay.want: lay.want + lay.W])
