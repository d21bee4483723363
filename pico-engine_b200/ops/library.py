"""The compiled kernel libraries and the declaration of their exported functions."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..csrc import build

P, I, F, LL, ULL = c_void_p, c_int, c_float, c_longlong, c_ulonglong

CORE_SOURCES = ("elementwise.cu", "linear_simt.cu", "attention_generic.cu", "sampling.cu", "linear_fused.cu", "gemm_tcgen05.cu")
# Kernels that no model needs unless it is asked for them: the allocation-free entry point and the split-K product it
# is built on (linear_mma.cu), and the two kernels for decode steps of 17 to 64 rows that the library's products with
# this library's small kernels between them still beat (linear_batch.cu: mma.sync with fused prologue and epilogues;
# gemm_splitk.cu: tcgen05 with K cut over a cluster).
EXTRA_SOURCES = ("linear_mma.cu", "linear_batch.cu", "gemm_splitk.cu")
HEAD_DIM_SOURCES = ("attention_decode.cu", "attention_prefill.cu", "attention_prefill_tcgen05.cu")      # compiled per head size

_SIGNATURES = {
    "pe_embed": [P, I, P, P, I, I, I, P],
    "pe_select_tokens": [P, P, P, I, P],
    "pe_rmsnorm": [P, P, P, I, F, P, I, I, I, P],
    "pe_add_rmsnorm": [P, P, I, P, I, F, P, I, I, I, P],
    "pe_swiglu": [P, P, I, I, I, P],
    "pe_residual_add": [P, P, I, LL, P],
    "pe_bias_add": [P, I, P, I, I, I, P],
    "pe_rope_store": [P, I, I, I, I, I, P, P, P, P, P, P, P, I, I, P],
    "pe_linear_simt": [P, I, P, I, P, I, P, I, I, I, I, P],
    "pe_attention_generic": [P, I, P, P, P, I, P, I, P, P, I, I, I, I, I, F, P],
    "pe_argmax": [P, P, I, I, P, P],
    "pe_sample": [P, P, I, I, F, I, F, ULL, P, P, P, P, P],
    "pe_gemm_tcgen05": [P, P, P, I, P, I, I, I, I, I, P, P],
    "pe_gemm_tcgen05_rope": [P, P, P, I, P, I, I, I, I, I, P, P, P, P, P, P, P, I, I, I, P, P],
    "pe_linear_fused": [P, P, P, I, F, P, P, I, P, I, I, I, I, P, P],
    "pe_norm_gate_up_swiglu": [P, P, I, F, P, P, I, I, I, P, P],
    "pe_norm_qkv_rope_store": [P, P, P, I, F, P, P, I, P, I, I, I, I, I, P, P, P, P, P, P, P, I, I, P, P],
}

_EXTRA_SIGNATURES = {
    "pe_gemm_splitk": [P, P, P, I, P, I, I, I, I, P, P],
    "pe_gemm_splitk_rope": [P, P, P, I, P, I, I, I, I, I, P, P, P, P, P, P, P, I, I, P, P],
    "pe_linear_mma": [P, P, P, I, P, I, I, I, I, P, P, P],
    "pe_linear_mma_splits": [I, I],
    "pe_linear_batch": [P, P, P, I, F, P, P, I, P, I, I, I, I, P, P],
    "pe_batch_norm_gate_up_swiglu": [P, P, I, F, P, P, I, I, I, P, P],
    "pe_batch_norm_qkv_rope_store": [P, P, I, F, P, P, I, P, I, I, I, I, I, P, P, P, P, P, P, P, I, I, P, P],
}

_HEAD_DIM_SIGNATURES = {
    "pe_attention_decode": [P, I, P, P, P, P, I, P, P, I, I, I, I, I, F, I, I, P, P],
    "pe_attention_decode_splits": [I, I, I, I, P],
    "pe_attention_prefill": [P, I, P, P, P, P, I, P, P, P, I, I, I, I, I, F, P],
    "pe_attention_prefill_tcgen05": [P, I, P, P, P, LL, P, I, P, I, I, I, I, I, I, F, P, P],
}

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_core = None
_by_head_dim = {}


def declare(lib: ctypes.CDLL, signatures: dict) -> None:
    for name, args in signatures.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


def core() -> ctypes.CDLL:
    """The library of the kernels every model needs; compiled at the first call."""
    global _core
    if _core is None:
        lib = build.load("core", CORE_SOURCES)
        declare(lib, _SIGNATURES)
        lib.pe_set_pdl(0 if os.environ.get("PICO_ENGINE_PDL", "1") == "0" else 1)
        lib.pe_draw_uniform.argtypes = [ULL, ULL, ULL]
        lib.pe_draw_uniform.restype = c_float
        lib.pe_argmax_scratch_bytes.argtypes = [I, I]
        lib.pe_argmax_scratch_bytes.restype = c_longlong
        lib.pe_sample_scratch_bytes.argtypes = [I, I]
        lib.pe_sample_scratch_bytes.restype = c_longlong
        _core = lib
    return _core


_extras = None


def extras() -> ctypes.CDLL:
    """The library of the kernels that are not on a model's default path; compiled at the first call."""
    global _extras
    if _extras is None:
        lib = build.load("extras", EXTRA_SOURCES)
        declare(lib, _EXTRA_SIGNATURES)
        lib.pe_set_pdl(0 if os.environ.get("PICO_ENGINE_PDL", "1") == "0" else 1)
        lib.pe_linear_mma_scratch_bytes.argtypes = [I, I, I]
        lib.pe_linear_mma_scratch_bytes.restype = c_longlong
        _extras = lib
    return _extras


def head_dim_sizes() -> range:
    """The head sizes the tensor-core attention kernels are compiled for on demand."""
    return range(16, 257, 16)


def for_head_dim(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention kernels compiled for one head size; compiled at the first call."""
    if head_dim not in head_dim_sizes():
        raise KernelError(f"head size {head_dim} is not taken: multiples of 16 from 16 to 256 are")
    lib = _by_head_dim.get(head_dim)
    if lib is None:
        lib = build.load(f"attention_hd{head_dim}", HEAD_DIM_SOURCES, {"PE_HEAD_DIM": str(head_dim)})
        declare(lib, _HEAD_DIM_SIGNATURES)
        lib.pe_set_pdl(0 if os.environ.get("PICO_ENGINE_PDL", "1") == "0" else 1)
        _by_head_dim[head_dim] = lib
    return lib


LAUNCHES = [0]      # kernels of this library launched so far (a captured launch counts once, when it is captured)


def check(code: int, name: str, kernels: int = 1) -> None:
    if code == 0:
        LAUNCHES[0] += kernels
        return
    if code == 10001:
        raise KernelError(f"{name}: sizes or dtypes that this kernel does not take")
    raise KernelError(f"{name}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"this library computes on CUDA devices only, not on {device}")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available, and this library has no CPU implementation")
    return device


def stream_ptr() -> int:
    """The raw handle of torch's current CUDA stream (the quick way: no Stream object is made)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())
