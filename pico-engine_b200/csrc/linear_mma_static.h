// pe_linear_mma_static: the small-M tensor-core product of linear_mma.cu for callers that
// must not allocate device memory.
//
// This entry point has no counterpart in pico-engine (which leaves every product to torch and
// its caching allocator); it exists for programs that embed this library but cannot let it,
// or anything it calls, reach cudaMalloc:
//   * a host application that has handed the whole device to its own memory pool and treats
//     any further driver allocation as an error (or would simply see it fail: no memory is left);
//   * a step that runs under a fixed memory budget that was negotiated before it started, where
//     an allocation at an arbitrary later moment can break a neighbour's guarantee;
//   * a latency-critical loop in which cudaMalloc's implicit device-wide synchronisation, or the
//     first-touch cost of fresh memory, is not acceptable.
// The ordinary entry point, pe_linear_mma, takes its scratch (the per-range partial sums and
// the tickets of the K ranges) from the caller, and this library's Python side gets that from
// torch's allocator.  Here the scratch is a fixed array inside the library instead:
//
//   out[M, N] = A[M, K] . W[N, K]^T (+ bias),  A and W bfloat16, M <= 64, K a multiple of 8
//   epilogue 0: out is float32;  1: out is bfloat16;  2: float32 out += result
//   bias: null, or N values of dtype bias_dtype (0 float32, 1 bfloat16)
//
// Limits and rules
//   * The array is PE_STATIC_SCRATCH_BYTES (1 MiB) of partial sums plus PE_STATIC_TICKETS
//     (1024) tickets.  It is part of the loaded library image: every GPU on which the library
//     is used holds it from the first use until the process exits, used or not.
//   * A product whose partial sums (ranges * M * N * 4 bytes, ranges = pe_linear_mma_splits(N, K))
//     or whose tickets (ceil(N / 16), only when ranges > 1) do not fit is refused with
//     PE_ERR_STATIC_TOO_LARGE before anything is launched; nothing larger is ever attempted.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it.  That first call is the set-up: make it before any
//     stream capture begins.
//   * All calls share the one array, and it keeps what the last call left.  The tickets must be
//     zero when a launch starts; each call clears them on its stream before it launches.  Two
//     calls that overlap on the GPU (different streams, or different host threads without
//     ordering) race on the array and give wrong sums: order them, e.g. by using one stream.
//   * No cudaMalloc, cudaFree or allocating library routine is called, here or in the kernel.
//
// Returns 0, a cudaError_t value, PE_ERR_UNSUPPORTED (10001) for shapes the kernel does not
// take at all, or PE_ERR_STATIC_TOO_LARGE (10002).
#pragma once

#define PE_STATIC_SCRATCH_BYTES (1u << 20)
#define PE_STATIC_TICKETS 1024u
#define PE_ERR_STATIC_TOO_LARGE 10002

#ifdef __cplusplus
extern "C" {
#endif

int pe_linear_mma_static(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                         int M, int N, int K, void* stream);

#ifdef __cplusplus
}
#endif
