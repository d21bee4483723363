"""RMSNorm."""
from __future__ import annotations

from ..config.specs import RMSNormSpec
from ..ops import kernels
from ..weights.loader import ParamSpec
from .base import Norm, register_norm


@register_norm(RMSNormSpec)
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w in float32 (pico-engine src/pico_engine/kernels.py:14-23).
    The weight stays in the dtype it was stored in."""

    def __init__(self, spec: RMSNormSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.weight = None
        self.eps = spec.eps

    def expected_tensors(self):
        return {self.spec.weight: ParamSpec((self.spec.size,), init="one_plus_normal")}

    def take_tensors(self, get):
        self.weight = get(self.spec.weight)

    def forward(self, x, out_dtype, rows_index=None):
        return kernels.rmsnorm(x, self.weight, self.eps, out_dtype, rows_index)

    def add_forward(self, x, y, out_dtype):
        return kernels.add_rmsnorm(x, y, self.weight, self.eps, out_dtype)
