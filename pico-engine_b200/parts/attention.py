"""Grouped-query softmax attention over the key/value cache."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed
from ..config.specs import ConfigError, GQAAttentionSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import POSITIONS, Mixer, build_part, register_mixer


@register_mixer(GQAAttentionSpec)
class GQAAttention(Mixer):
    """pico-engine src/pico_engine/model.py:175-213: one product for q, k and v on concatenated
    weights (model.py:85-94, 177), position encoding of q and k, keys and values into the cache,
    attention over the cache, output projection added to the residual stream (model.py:213).

    With ``owns_cache`` false the layer reads the cache of another schedule entry: it projects
    and rotates its queries, writes nothing, and sees that entry's keys and values.
    """

    def __init__(self, spec: GQAAttentionSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.n_heads % spec.n_kv_heads:
            raise ConfigError(f"{spec.n_heads} query heads cannot share {spec.n_kv_heads} key/value heads evenly")
        if spec.head_dim % 16 or not 16 <= spec.head_dim <= 256:
            raise ConfigError(f"head_dim {spec.head_dim} is not taken: the attention kernels take multiples of 16 "
                              f"from 16 to 256")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError(f"window {spec.window} must be positive")
        self.position = build_part(POSITIONS, "position encoding", spec.position, dtype, device)
        self.w_qkv = self.b_qkv = self.w_o = None

    # ------------------------------------------------------------------ weights
    def _names(self):
        s = self.spec
        return [s.prefix + n for n in (s.q_name, s.k_name, s.v_name, s.o_name)]

    def expected_tensors(self):
        s = self.spec
        q, k, v, o = self._names()
        out = {q + ".weight": ParamSpec((s.n_heads * s.head_dim, s.hidden)),
               k + ".weight": ParamSpec((s.n_kv_heads * s.head_dim, s.hidden)),
               v + ".weight": ParamSpec((s.n_kv_heads * s.head_dim, s.hidden)),
               o + ".weight": ParamSpec((s.hidden, s.n_heads * s.head_dim))}
        if s.qkv_bias:
            out.update({q + ".bias": ParamSpec((s.n_heads * s.head_dim,)),
                        k + ".bias": ParamSpec((s.n_kv_heads * s.head_dim,)),
                        v + ".bias": ParamSpec((s.n_kv_heads * s.head_dim,))})
        out.update(self.position.expected_tensors())
        return out

    def take_tensors(self, get):
        q, k, v, o = self._names()
        self.w_qkv = torch.cat([get(q + ".weight"), get(k + ".weight"), get(v + ".weight")], dim=0).contiguous()
        if self.spec.qkv_bias:
            self.b_qkv = torch.cat([get(q + ".bias"), get(k + ".bias"), get(v + ".bias")]).contiguous()
        self.w_o = get(o + ".weight")
        self.position.take_tensors(get)

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    # ------------------------------------------------------------------ cache and step
    def cache_needs(self):
        s = self.spec
        return CacheNeeds(kv=KVNeed(s.n_kv_heads, s.head_dim, s.window))

    def _attend(self, h, ctx, cache_entry, owns_cache):
        from ..ops.linear import qkv_rope_store, qkv_rope_store_takes
        from .position import NoPosition, RotaryHalf
        s = self.spec
        kv = ctx.kv(cache_entry)
        if type(self.position) in (RotaryHalf, NoPosition) and qkv_rope_store_takes(h, self.w_qkv, self.b_qkv, s.head_dim):
            # many rows in bfloat16: projection, bias, rotation and cache write can be one tcgen05 kernel
            cos, sin = self._tables(ctx)
            q = qkv_rope_store(h, self.w_qkv, self.b_qkv, s.n_heads, s.n_kv_heads, s.head_dim, cos, sin, ctx.tok_pos,
                               ctx.tok_row, kv.k if owns_cache else None, kv.v if owns_cache else None, kv.table, kv.stride)
            if q is not None:
                return kernels.attention(q, q.shape[1], s.n_heads, s.n_kv_heads, s.head_dim, kv.k, kv.v, kv.table,
                                         kv.stride, ctx.tok_pos, ctx.tok_row, s.window, s.scale, ctx, own_rows_only=owns_cache)
        qkv = linear(h, self.w_qkv, self.b_qkv, out_dtype=ctx.dtype)
        self.position.rotate_and_store(qkv, s.n_heads, s.n_kv_heads, s.head_dim, ctx, kv if owns_cache else None)
        return kernels.attention(qkv, qkv.shape[1], s.n_heads, s.n_kv_heads, s.head_dim, kv.k, kv.v, kv.table,
                                 kv.stride, ctx.tok_pos, ctx.tok_row, s.window, s.scale, ctx, own_rows_only=owns_cache)

    def _tables(self, ctx):
        """The rotary tables of this layer's position encoding (None, None where it has none), checked
        against the longest sequence of the step."""
        cos, sin = getattr(self.position, "cos", None), getattr(self.position, "sin", None)
        if cos is not None and ctx.max_context > cos.shape[0]:
            raise ValueError(f"a sequence reaches position {ctx.max_context - 1}, the rotary tables hold "
                             f"{cos.shape[0]} positions")
        return cos, sin

    def apply(self, h, ctx, entry, cache_entry, owns_cache):
        return linear(self._attend(h, ctx, cache_entry, owns_cache), self.w_o, out_dtype=ctx.dtype)

    def _fused(self, x, norm, ctx) -> bool:
        """Decoding a few sequences in bfloat16: norm, projection, position encoding and cache
        write are one kernel (csrc/linear_fused.cu)."""
        from .norm import RMSNorm
        from .position import NoPosition, RotaryHalf
        return (ctx.dtype == torch.bfloat16 and type(norm) is RMSNorm and type(self.position) in (RotaryHalf, NoPosition)
                and (self.b_qkv is None or self.b_qkv.dtype in (torch.bfloat16, torch.float32))
                and kernels.decode_fused_takes(x.shape[0], self.w_qkv, x) and kernels.decode_fused_takes(x.shape[0], self.w_o))

    takes_pending = True

    def add_to(self, x, norm, ctx, entry, cache_entry, owns_cache):
        if self._fused(x, norm, ctx):
            ctx.settle(x)
            s = self.spec
            kv = ctx.kv(cache_entry)
            cos, sin = self._tables(ctx)
            q = kernels.norm_qkv_rope_store(x, norm.weight, norm.eps, self.w_qkv, self.b_qkv, s.n_heads, s.n_kv_heads,
                                            s.head_dim, cos, sin, ctx.tok_pos, ctx.tok_row,
                                            kv.k if owns_cache else None, kv.v if owns_cache else None, kv.table, kv.stride)
            # (an entry that reads another entry's cache may follow it closely: that entry's kernels wrote its rows)
            a = kernels.attention(q, q.shape[1], s.n_heads, s.n_kv_heads, s.head_dim, kv.k, kv.v, kv.table, kv.stride,
                                  ctx.tok_pos, ctx.tok_row, s.window, s.scale, ctx, own_rows_only=owns_cache)
            kernels.linear_fused(a, self.w_o, accumulate_into=x)
            return
        a = self._attend(ctx.normed(x, norm), ctx, cache_entry, owns_cache)
        linear(a, self.w_o, accumulate_into=x, defer_add=lambda y: ctx.defer_add(x, y))
