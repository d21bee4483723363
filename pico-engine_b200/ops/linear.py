"""out = a . w^T (+ bias), stored or added into the float32 residual stream, possibly fused with what
follows it in a layer: the choice of kernel for a matrix product.

* bfloat16 activations and weights, up to 16 rows (decoding): the tensor-core weight-streaming
  kernel with bias and residual in its epilogue, ``csrc/linear_fused.cu``.
* bfloat16, more rows (larger decode batches, prompts): either this library's tcgen05 kernel
  (``csrc/gemm_tcgen05.cu``) with the step that follows the product in its epilogue (bias, residual
  sum, SwiGLU, or bias + rotation + cache write), or the library product (cuBLAS through ``torch.mm``,
  which is where pico-engine uses a library too: src/pico_engine/model.py:177, 213, 223, 235) followed by
  this library's kernel for that step.  Which of the two is faster depends on the sizes (the library
  has tile shapes and TMA multicast that this kernel has not; this kernel saves a pass over the product),
  so the first time a product of some shape is asked for, both are timed on the device, a few replays of
  a captured CUDA graph each, and the faster one is remembered (``Choice``).  ``PICO_ENGINE_GEMM=tcgen05``
  or ``=library`` fixes the choice instead.
* anything else (the float32 engine; weights that were stored in float32): float32
  multiply-adds on the CUDA cores, ``csrc/linear_simt.cu``.
"""
from __future__ import annotations

import gc
import os
from typing import Callable, Dict, Optional, Tuple

import torch

from . import kernels

_FORCED = os.environ.get("PICO_ENGINE_GEMM", "auto").lower()      # auto | tcgen05 | library
_CHOICES_FILE = os.environ.get("PICO_ENGINE_GEMM_CHOICES")        # a JSON file of earlier decisions (Choice.save) to start from


class Choice:
    """Which implementation runs a product, by (what follows it, row bucket, N, K): decided once by
    timing both, then remembered for the life of the process."""

    table: Dict[Tuple, str] = {}
    timings: Dict[Tuple, Tuple[float, float]] = {}       # key -> (tcgen05 us, library us), for reports

    @classmethod
    def save(cls, path: str) -> None:
        """Write the decisions made so far; ``PICO_ENGINE_GEMM_CHOICES=path`` makes a later process start from them
        (no timing for shapes that are listed: a run under a profiler, whose clock is not the device's, keeps the
        choices of a plain run; a service skips the first-use measurements)."""
        import json
        with open(path, "w") as f:
            json.dump({"|".join(str(x) for x in k): v for k, v in cls.table.items()}, f, indent=1, sort_keys=True)

    @classmethod
    def load(cls, path: str) -> None:
        import json
        with open(path) as f:
            for k, v in json.load(f).items():
                if v not in ("tcgen05", "library"):
                    raise ValueError(f"{path}: the choice for {k} must be tcgen05 or library, not {v!r}")
                parts = k.split("|")
                cls.table[(parts[0],) + tuple(int(x) for x in parts[1:])] = v

    @staticmethod
    def bucket(rows: int) -> int:
        """Row counts that share a decision: powers of two from 32 on."""
        b = 32
        while b < rows:
            b *= 2
        return b

    # A step of many rows is launched kernel by kernel from Python, at 10 to 13 us of host time a launch
    # (measured: 220 launches of a 2,048-token step of the Qwen2.5-0.5B shape take 3.2 ms), which is as long as
    # the device needs for them: a launch that the fused kernel saves is worth about this much there.  Steps of up
    # to CAPTURED_ROWS rows are decode steps, replayed from a graph, where only device time counts.
    HOST_US_PER_LAUNCH = 6.0
    CAPTURED_ROWS = 128

    @classmethod
    def pick(cls, key: Tuple, own: Callable[[], object], library: Callable[[], object], launches_saved: int = 0) -> str:
        """"tcgen05" or "library" for ``key``; the two callables run the product on scratch operands
        of the key's sizes; ``launches_saved``: how many launches fewer the fused kernel is.  While a CUDA
        graph is being captured nothing can be timed: the library product runs, and the question is asked
        again outside a capture."""
        got = cls.table.get(key)
        if got is not None:
            return got
        if _FORCED in ("tcgen05", "library"):
            cls.table[key] = _FORCED
            return _FORCED
        if torch.cuda.is_current_stream_capturing():
            return "library"
        t_own, t_lib = _device_time(own), _device_time(library)
        cls.timings[key] = (t_own, t_lib)
        host = cls.HOST_US_PER_LAUNCH * launches_saved if key[1] > cls.CAPTURED_ROWS else 0.0
        cls.table[key] = "tcgen05" if t_own < t_lib + host else "library"
        return cls.table[key]


if _CHOICES_FILE and os.path.isfile(_CHOICES_FILE):
    Choice.load(_CHOICES_FILE)


def _device_time(fn: Callable[[], object], calls: int = 6, replays: int = 3) -> float:
    """Microseconds a call of ``fn`` takes on the device: ``calls`` of them in one captured graph (no host
    in between), the best of ``replays`` replays."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    collecting = gc.isenabled()
    gc.disable()                                 # nothing that owns device resources is freed in the middle of a capture
    try:
        with torch.cuda.stream(side):
            fn()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(calls):
                    fn()
    finally:
        if collecting:
            gc.enable()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1000.0 / calls)
    return best


def _scratch_rows(rows: int, cols: int, dtype, device) -> torch.Tensor:
    return torch.zeros(rows, cols, dtype=dtype, device=device)


def _takes_tcgen05(a: torch.Tensor, w: torch.Tensor) -> bool:
    return a.shape[0] > kernels.FUSED_MAX_ROWS and kernels.gemm_tcgen05_takes(a, w)


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
        if bias is None and accumulate_into is None and out_dtype == torch.float32:
            return torch.mm(a, w.t(), out_dtype=torch.float32)   # the logits: the library's float32 accumulator as it is
        if accumulate_into is not None and bias is None and _takes_tcgen05(a, w):
            key = ("accumulate", Choice.bucket(M), w.shape[0], w.shape[1])
            if key not in Choice.table:
                rows = Choice.bucket(M)
                sa, sx = _scratch_rows(rows, a.shape[1], a.dtype, a.device), _scratch_rows(rows, w.shape[0], torch.float32, a.device)
                Choice.pick(key, lambda: kernels.gemm_tcgen05(sa, w, accumulate_into=sx),
                            lambda: kernels.residual_add(sx, torch.mm(sa, w.t())))
            if Choice.table.get(key) == "tcgen05":
                return kernels.gemm_tcgen05(a, w, accumulate_into=accumulate_into)
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


def gate_up_swiglu(h: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(h Wg^T) * (h Wu^T) [T, I] for h [T, K] and w_gate_up = [Wg; Wu] [2I, K]: one tcgen05 kernel with the
    activation in its epilogue, or the product followed by the SwiGLU kernel."""
    if h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and _takes_tcgen05(h, w_gate_up) \
            and w_gate_up.shape[0] % 16 == 0:
        M = h.shape[0]
        key = ("swiglu", Choice.bucket(M), w_gate_up.shape[0], w_gate_up.shape[1])
        if key not in Choice.table:
            sh = _scratch_rows(Choice.bucket(M), h.shape[1], h.dtype, h.device)
            Choice.pick(key, lambda: kernels.gemm_tcgen05(sh, w_gate_up, swiglu=True),
                        lambda: kernels.swiglu(torch.mm(sh, w_gate_up.t())), launches_saved=1)
        if Choice.table.get(key) == "tcgen05":
            return kernels.gemm_tcgen05(h, w_gate_up, swiglu=True)
    return kernels.swiglu(linear(h, w_gate_up, out_dtype=h.dtype))


def qkv_rope_store_takes(h: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], head_dim: int) -> bool:
    return (h.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and head_dim in kernels.GEMM_ROPE_HEAD_DIMS
            and _takes_tcgen05(h, w_qkv) and (b_qkv is None or b_qkv.dtype in (torch.bfloat16, torch.float32)))


def qkv_rope_store(h: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_row: torch.Tensor,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
                   table_stride: int) -> Optional[torch.Tensor]:
    """Rotated queries [T, n_q * head_dim] with keys and values written to their cache pages, in one tcgen05
    kernel; or None where the product followed by the rotation kernel is faster (the caller then runs those)."""
    M = h.shape[0]
    key = ("rope", Choice.bucket(M), w_qkv.shape[0], w_qkv.shape[1], head_dim)
    if key not in Choice.table:
        rows = Choice.bucket(M)
        sh = _scratch_rows(rows, h.shape[1], h.dtype, h.device)
        pos = torch.zeros(rows, dtype=torch.int32, device=h.device)
        # timed without the cache write on both sides (a scratch cache would have to be as large as the real one)
        own = lambda: kernels.gemm_qkv_rope_store(sh, w_qkv, b_qkv, n_q, n_kv, head_dim, cos, sin, pos, pos, None, None, None, 0)

        def library():
            y = linear(sh, w_qkv, b_qkv, out_dtype=h.dtype)
            kernels.rope_store(y, n_q, n_kv, head_dim, cos, sin, pos, pos, None, None, None, 0)
        Choice.pick(key, own, library, launches_saved=1)
    if Choice.table.get(key) != "tcgen05":
        return None
    return kernels.gemm_qkv_rope_store(h, w_qkv, b_qkv, n_q, n_kv, head_dim, cos, sin, tok_pos, tok_row, k_pool, v_pool,
                                       block_table, table_stride)
