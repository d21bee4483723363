"""The allocation-free entry point ``pe_linear_mma_static`` (csrc/linear_mma_static.h), called
through its exported C symbol as an embedding program would, against the ordinary entry point.

It serves hosts that cannot let this library allocate device memory (a process that has given
the whole GPU to its own pool, a step running under a fixed memory budget, a loop that cannot
afford cudaMalloc's synchronisation).  This file is collected last, so a run that stops at the
first failure has run every other test before it.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE, UNSUPPORTED = 10002, 10001


@pytest.fixture(scope="module")
def static_entry():
    from pico_engine.ops.library import extras
    fn = extras().pe_linear_mma_static                 # the exported symbol; nothing in the package wraps it
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, I, P, I, I, I, I, P]
    fn.restype = I
    return fn


def operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    return a, w, b


@pytest.mark.parametrize("M,N,K", [(8, 896, 4864), (64, 1152, 896), (1, 896, 896), (13, 9728, 896)])
def test_two_calls_in_a_row_equal_the_ordinary_entry_point(static_entry, M, N, K):
    from pico_engine.ops import kernels
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                                       # the second call finds what the first left behind
        a, w, b = operands(M, N, K, seed=10 * call + M)
        want = kernels.linear_mma(a, w, b, out_dtype=torch.float32)
        got = torch.empty(M, N, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = static_entry(a.data_ptr(), w.data_ptr(), b.data_ptr(), 1, got.data_ptr(), 0, M, N, K, stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before          # torch's allocator was not asked either
        torch.cuda.synchronize()
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), float((got - want).abs().max())
        exact = a.double().cpu() @ w.double().cpu().T + b.double().cpu()
        assert torch.allclose(got.double().cpu(), exact, atol=1e-4, rtol=1e-4)
    # adding into a float32 tensor, as the residual stream is updated
    a, w, b = operands(M, N, K, seed=99)
    x = torch.randn(M, N, device="cuda")
    want = kernels.linear_mma(a, w, None, accumulate_into=x.clone())
    got = x.clone()
    assert static_entry(a.data_ptr(), w.data_ptr(), None, 0, got.data_ptr(), 2, M, N, K, stream) == 0
    torch.cuda.synchronize()
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)


def test_sizes_beyond_the_fixed_array_are_refused(static_entry):
    from pico_engine.ops.library import extras
    lib = extras()
    lib.pe_linear_mma_scratch_bytes.argtypes = [ctypes.c_int] * 3
    lib.pe_linear_mma_scratch_bytes.restype = ctypes.c_longlong
    M, N, K = 64, 1152, 2048                                     # five K ranges of 64 x 1152 sums: 1.4 MiB, the array holds 1 MiB
    assert lib.pe_linear_mma_scratch_bytes(M, N, K) > 1 << 20
    assert lib.pe_linear_mma_scratch_bytes(8, N, K) < 1 << 20
    a, w, _ = operands(M, N, K, seed=1)
    out = torch.full((M, N), 7.0, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert static_entry(a.data_ptr(), w.data_ptr(), None, 0, out.data_ptr(), 0, M, N, K, stream) == TOO_LARGE
    assert static_entry(a.data_ptr(), w.data_ptr(), None, 0, out.data_ptr(), 0, 65, N, K, stream) == UNSUPPORTED
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0   # nothing was launched
    assert static_entry(a.data_ptr(), w.data_ptr(), None, 0, out.data_ptr(), 0, 8, N, K, stream) == 0   # fewer rows fit
    torch.cuda.synchronize()
    assert torch.allclose(out[:8].cpu().double(), a[:8].double().cpu() @ w.double().cpu().T, atol=1e-4, rtol=1e-4)
