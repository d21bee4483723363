"""Position encodings applied to the query and key heads before keys enter the cache."""
from __future__ import annotations

import torch

from ..config.specs import NoPositionSpec, RotaryHalfSpec
from ..ops import kernels
from .base import Position, register_position


@register_position(RotaryHalfSpec)
class RotaryHalf(Position):
    """Rotate-half rotary encoding (pico-engine src/pico_engine/model.py:75-79, kernels.py:37-47).

    The cos/sin tables are computed once, in float32 on the host with the project's own
    formula, for as many positions as a sequence can have; the kernel reads them by position.
    """

    def __init__(self, spec: RotaryHalfSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.cos = self.sin = None

    def prepare(self, max_positions: int) -> None:
        hd = self.spec.head_dim
        inv_freq = 1.0 / (self.spec.theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
        angles = torch.arange(max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        self.cos = angles.cos().to(self.device).contiguous()
        self.sin = angles.sin().to(self.device).contiguous()

    def weights(self):
        return []                      # the tables are read by position, a few rows a step

    def rotate_and_store(self, qkv, n_q, n_kv, head_dim, ctx, kv):
        if ctx.max_context > self.cos.shape[0]:
            raise ValueError(f"a sequence reaches position {ctx.max_context - 1}, the rotary tables hold "
                             f"{self.cos.shape[0]} positions")
        kernels.rope_store(qkv, n_q, n_kv, head_dim, self.cos, self.sin, ctx.tok_pos, ctx.tok_row,
                           None if kv is None else kv.k, None if kv is None else kv.v,
                           None if kv is None else kv.table, 0 if kv is None else kv.stride)


@register_position(NoPositionSpec)
class NoPosition(Position):
    """Keys and queries as projected; only the cache write happens."""

    def rotate_and_store(self, qkv, n_q, n_kv, head_dim, ctx, kv):
        if kv is not None:
            kernels.rope_store(qkv, n_q, n_kv, head_dim, None, None, ctx.tok_pos, ctx.tok_row, kv.k, kv.v,
                               kv.table, kv.stride)
