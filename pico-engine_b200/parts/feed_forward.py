"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from ..config.specs import SwiGLUSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import FeedForward, register_feed_forward


@register_feed_forward(SwiGLUSpec)
class SwiGLU(FeedForward):
    """down(silu(gate(h)) * up(h)) with gate and up as one product on concatenated weights
    (pico-engine src/pico_engine/model.py:95-98, 222-235; kernels.py:62-74)."""

    def __init__(self, spec: SwiGLUSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.w_gate_up = self.w_down = None

    def expected_tensors(self):
        s = self.spec
        return {s.prefix + s.gate_name + ".weight": ParamSpec((s.intermediate, s.hidden)),
                s.prefix + s.up_name + ".weight": ParamSpec((s.intermediate, s.hidden)),
                s.prefix + s.down_name + ".weight": ParamSpec((s.hidden, s.intermediate))}

    def take_tensors(self, get):
        s = self.spec
        self.w_gate_up = torch.cat([get(s.prefix + s.gate_name + ".weight"),
                                    get(s.prefix + s.up_name + ".weight")], dim=0).contiguous()
        self.w_down = get(s.prefix + s.down_name + ".weight")

    def _activation(self, h, ctx):
        from ..ops.linear import gate_up_swiglu
        return gate_up_swiglu(h, self.w_gate_up)

    def apply(self, h, ctx):
        return linear(self._activation(h, ctx), self.w_down, out_dtype=ctx.dtype)

    takes_pending = True

    def add_to(self, x, norm, ctx):
        from .norm import RMSNorm
        if (ctx.dtype == torch.bfloat16 and type(norm) is RMSNorm and self.spec.intermediate % 8 == 0
                and kernels.decode_fused_takes(x.shape[0], self.w_gate_up, x) and kernels.decode_fused_takes(x.shape[0], self.w_down)):
            # decoding a few sequences: norm, gate and up products and the activation are one kernel
            ctx.settle(x)
            act = kernels.norm_gate_up_swiglu(x, norm.weight, norm.eps, self.w_gate_up)
            kernels.linear_fused(act, self.w_down, accumulate_into=x)
            return
        linear(self._activation(ctx.normed(x, norm), ctx), self.w_down, accumulate_into=x,
               defer_add=lambda y: ctx.defer_add(x, y))
