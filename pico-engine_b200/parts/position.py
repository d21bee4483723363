"""Position encodings applied to the query and key heads before keys enter the cache."""
from __future__ import annotations

import torch

from ..config.specs import NoPositionSpec, RotaryHalfSpec
from ..ops import kernels
from .base import Position, register_position


_TABLES = {}      # (head_dim, theta, device) -> (cos, sin) for the most positions asked for so far


def rotary_tables(head_dim: int, theta: float, max_positions: int, device):
    """cos and sin [positions >= max_positions, head_dim / 2] float32 on ``device``, one pair per (head size, base,
    device) for all layers and engines of the process: the layers of a model have the same tables, and a decode
    step that reads the same few rows in every layer finds them in cache."""
    key = (head_dim, float(theta), str(device))
    have = _TABLES.get(key)
    if have is None or have[0].shape[0] < max_positions:
        inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
        angles = torch.arange(max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        have = _TABLES[key] = (angles.cos().to(device).contiguous(), angles.sin().to(device).contiguous())
    return have


@register_position(RotaryHalfSpec)
class RotaryHalf(Position):
    """Rotate-half rotary encoding (pico-engine src/pico_engine/model.py:75-79, kernels.py:37-47).

    The cos/sin tables are computed once, in float32 on the host with the project's own
    formula, for as many positions as a sequence can have; the kernel reads them by position.
    All layers with the same head size and base share one pair of tables (``rotary_tables``).
    """

    def __init__(self, spec: RotaryHalfSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.cos = self.sin = None

    def prepare(self, max_positions: int) -> None:
        self.cos, self.sin = rotary_tables(self.spec.head_dim, self.spec.theta, max_positions, self.device)

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
