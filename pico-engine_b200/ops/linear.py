"""out = a . w^T (+ bias), stored or added into the float32 residual stream: the choice of
kernel for a matrix product.

* bfloat16 activations and weights, up to 16 rows (decoding): the tensor-core weight-streaming
  kernel with bias and residual in its epilogue, ``csrc/linear_fused.cu``.
* bfloat16, more rows (larger decode batches, prompts): the library product (cuBLAS through
  ``torch.mm``), which is where pico-engine uses a library too (src/pico_engine/model.py:177,
  213, 223, 235), followed by this library's bias or residual kernel; or, where that is faster,
  the tcgen05 kernel of ``csrc/gemm_tcgen05.cu`` with the residual sum in its epilogue.
  (``csrc/linear_mma.cu`` takes up to 64 rows, but from 17 rows on the library is two to
  three times faster on a B200: 5.7 us against 15.4 us for 64 x 9728 x 896.)
* anything else (the float32 engine; weights that were stored in float32): float32
  multiply-adds on the CUDA cores, ``csrc/linear_simt.cu``.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import kernels

# A product with a small weight that ends in the residual sum runs on this library's tcgen05 kernel,
# which adds into the stream in its epilogue: there the library's product plus a separate pass over the
# result costs more (17 us against 30 us for 2048 x 896 x 896).  Larger products are still faster in cuBLAS.
TCGEN05_MAX_WEIGHT = 1 << 20
TCGEN05_MAX_ROWS = 4096
TCGEN05_MIN_ROWS = 512      # below this its 128-row tiles leave most SMs without work


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
           defer_add: Optional[Callable[[torch.Tensor], None]] = None) -> torch.Tensor:
    """``defer_add``: where the product comes from the library and its sum into ``accumulate_into`` would be a
    pass of its own, the product is handed to this function instead, and the caller adds it later (with the
    norm that follows, in one pass)."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        M = a.shape[0]
        if kernels.fused_takes(M, w, a):
            return kernels.linear_fused(a, w, bias, out_dtype, accumulate_into)
        if (accumulate_into is not None and bias is None and w.numel() <= TCGEN05_MAX_WEIGHT and TCGEN05_MIN_ROWS <= M <= TCGEN05_MAX_ROWS
                and kernels.gemm_tcgen05_takes(a, w)):
            return kernels.gemm_tcgen05(a, w, accumulate_into=accumulate_into)
        if bias is None and accumulate_into is None and out_dtype == torch.float32:
            return torch.mm(a, w.t(), out_dtype=torch.float32)   # the logits: the library's float32 accumulator as it is
        if bias is not None and bias.dtype == a.dtype:
            y = torch.addmm(bias, a, w.t())                  # the library adds the bias in its epilogue
        else:
            y = torch.mm(a, w.t())
            if bias is not None:
                kernels.bias_add(y, bias)
        if accumulate_into is not None:
            if defer_add is not None:
                defer_add(y)
                return accumulate_into
            return kernels.residual_add(accumulate_into, y)
        return y if (out_dtype or a.dtype) == y.dtype else y.to(out_dtype)
    return kernels.linear_simt(a, w, bias, out_dtype, accumulate_into)
