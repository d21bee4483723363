"""Interfaces of the parts of a layer, the context a step hands them, and the registries that
map a part's description (``config.specs``) to its implementation.

No part knows which model it is in: it gets its sizes and constants from its spec, its
tensors by the names in its spec, and everything about the running step from the
:class:`StepContext`.

A rule for parts that write the key/value cache: the decode attention kernel (``kernels.attention`` for single
tokens in bfloat16) starts copying cache pages while the two kernels launched before it may still run, and
fetches again only each token's own newest row.  A part that writes other rows of a cache shortly before that
cache is attended to (within two launches) passes ``own_rows_only=False`` to ``kernels.attention``; the
attention part does so for a schedule entry that reads another entry's cache (``cache_of``).

Interfaces
----------
Norm          ``forward(x_f32 [T,H], out_dtype, rows_index=None) -> [rows,H]``; optionally
              ``add_forward(x, y, out_dtype)``: x += y and the norm in one pass
Position      ``prepare(max_positions)``; ``rotate_and_store(qkv, n_q, n_kv, head_dim, ctx, kv)``
Mixer         ``cache_needs()``; ``prepare(max_positions)``; ``apply(h, ctx, entry, cache_entry,
              owns_cache) -> y``; optionally ``add_to(x, norm, ctx, ...)`` fused
FeedForward   ``apply(h, ctx) -> y``; optionally ``add_to(x, norm, ctx)`` fused
Arrangement   ``run(layer, x, ctx, entry, cache_entry, owns_cache)``: updates ``x`` in place
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..cache import CacheNeeds
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import ParamSpec


@dataclass
class KVView:
    """Keys and values of one schedule entry for the running step."""
    k: torch.Tensor               # [page, kv head, PAGE, head_dim]
    v: torch.Tensor
    table: torch.Tensor           # int32 [B, stride]: physical page of each logical page of each batch row
    stride: int
    window: Optional[int]


@dataclass
class StepContext:
    """Everything a part may know about the running step.

    The step runs ``T`` tokens of ``B`` sequences, packed sequence after sequence.  Token t
    belongs to batch row ``tok_row[t]`` and stands at position ``tok_pos[t]`` of its sequence; row b's
    tokens are ``row_first[b] .. row_first[b + 1] - 1``.  The device arrays are what a kernel needs to
    find its rows, also inside a captured graph, where the host lists (``lens``, ``starts``,
    ``slot_ids``) are those of the step that was captured and must not be read.  A captured step
    of a fixed number of rows may carry idle rows: they bring one token at position 0 of the cache's idle
    slot, and nobody reads what they produce.
    """
    T: int
    B: int
    dtype: torch.dtype                    # dtype of activations and cache
    device: torch.device
    tok_pos: torch.Tensor                 # int32 [T], device
    tok_row: torch.Tensor                 # int32 [T], device
    slots: torch.Tensor                   # int32 [B], device: sequence slot of each batch row
    row_first: torch.Tensor               # int32 [B + 1], device: packed index of each row's first token; row_first[B] = T
    row_lens: torch.Tensor                # int32 [B], device: tokens each row brings in this step
    slot_ids: List[int]                   # the slots on the host
    lens: List[int]                       # tokens of each row in this step (host)
    starts: List[int]                     # position of each row's first token (host)
    one_token_each: bool                  # every row brings exactly one token
    cache: object                         # cache.Cache
    tables: Dict[int, torch.Tensor] = field(default_factory=dict)    # group -> int32 [B, stride]
    max_context: int = 0                  # upper bound of any row's length after the step
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)   # named buffers that live as long as the step
    pending: Optional[torch.Tensor] = None  # a product [T, hidden] that still has to be added to the residual stream

    # A part whose product comes out of the library may leave the sum into the residual stream pending, so
    # that the norm that follows does both in one pass.  Whoever reads the stream first settles it: parts
    # that declare ``takes_pending`` through ``normed``, everyone else through the arrangement.
    def defer_add(self, x: torch.Tensor, y: torch.Tensor) -> None:
        self.settle(x)
        self.pending = y

    def settle(self, x: torch.Tensor) -> None:
        if self.pending is not None:
            from ..ops import kernels
            y, self.pending = self.pending, None
            kernels.residual_add(x, y.contiguous())

    def normed(self, x: torch.Tensor, norm: "Norm") -> torch.Tensor:
        """norm(x) in the step's dtype, after what is pending has been added to x."""
        if self.pending is None:
            return norm.forward(x, self.dtype)
        y, self.pending = self.pending, None
        return norm.add_forward(x, y.contiguous(), self.dtype)

    def kv(self, cache_entry: int) -> KVView:
        g = self.cache.group_of[cache_entry]
        k, v = self.cache.pools(cache_entry)
        t = self.tables[g]
        return KVView(k, v, t, t.shape[1], self.cache.groups[g].need.window)

    def state(self, cache_entry: int) -> Optional[torch.Tensor]:
        """[slot, elems] float32; row ``slots[b]`` is batch row b's state."""
        return self.cache.state_of(cache_entry)


class Part:
    def __init__(self, spec: PartSpec, dtype: torch.dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def expected_tensors(self) -> Dict[str, ParamSpec]:
        return {}

    def take_tensors(self, get: Callable[[str], torch.Tensor]) -> None:
        pass

    def prepare(self, max_positions: int) -> None:
        """Called once before the first step, with the longest sequence the cache can hold."""

    def weights(self) -> List[torch.Tensor]:
        """The tensors a step reads in full (for traffic accounting)."""
        return [v for v in vars(self).values() if isinstance(v, torch.Tensor)]


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, y: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """x += y in place, then forward(x); norms override this to do both in one pass."""
        from ..ops import kernels
        kernels.residual_add(x, y)
        return self.forward(x, out_dtype)


class Position(Part):
    def rotate_and_store(self, qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, ctx: StepContext,
                         kv: Optional[KVView]) -> None:
        raise NotImplementedError


class Mixer(Part):
    takes_pending = False      # True: add_to copes with a sum that is still pending (StepContext.normed / settle)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def apply(self, h: torch.Tensor, ctx: StepContext, entry: int, cache_entry: int, owns_cache: bool) -> torch.Tensor:
        raise NotImplementedError

    def add_to(self, x: torch.Tensor, norm: Norm, ctx: StepContext, entry: int, cache_entry: int, owns_cache: bool) -> None:
        """x += apply(norm(x)); parts override this to fuse the norm and the residual sum."""
        from ..ops import kernels
        kernels.residual_add(x, self.apply(norm.forward(x, ctx.dtype), ctx, entry, cache_entry, owns_cache).contiguous())


class FeedForward(Part):
    takes_pending = False

    def apply(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def add_to(self, x: torch.Tensor, norm: Norm, ctx: StepContext) -> None:
        from ..ops import kernels
        kernels.residual_add(x, self.apply(norm.forward(x, ctx.dtype), ctx).contiguous())


# ------------------------------------------------------------------ registries

NORMS: Dict[type, type] = {}
POSITIONS: Dict[type, type] = {}
MIXERS: Dict[type, type] = {}
FEED_FORWARDS: Dict[type, type] = {}
ARRANGEMENTS: Dict[str, Callable] = {}


def _register(table: Dict[type, type], spec_class: type):
    def deco(cls):
        table[spec_class] = cls
        return cls
    return deco


def register_norm(spec_class: type):
    return _register(NORMS, spec_class)


def register_position(spec_class: type):
    return _register(POSITIONS, spec_class)


def register_mixer(spec_class: type):
    return _register(MIXERS, spec_class)


def register_feed_forward(spec_class: type):
    return _register(FEED_FORWARDS, spec_class)


def register_arrangement(name: str):
    def deco(fn):
        ARRANGEMENTS[name] = fn
        return fn
    return deco


def build_part(table: Dict[type, type], kind: str, spec: PartSpec, dtype, device) -> Part:
    try:
        cls = table[type(spec)]
    except KeyError:
        known = ", ".join(sorted(c.__name__ for c in table)) or "none"
        raise ConfigError(f"no {kind} is registered for {type(spec).__name__}; registered: {known}") from None
    return cls(spec, dtype, device)
