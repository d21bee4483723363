// NOT ON THE GENERATION PATH: no step of the engine calls this kernel any more (up to 16 rows run linear_fused.cu,
// more rows gemm_tcgen05.cu or the library's product).  It is kept for the entry point that allocates nothing
// (pe_linear_mma_static at the end of this file, declared in linear_mma_static.h) and for the tests of both:
// tuning it speeds nothing up.
//
// out[M, N] = A[M, K] . W[N, K]^T (+ bias) for few rows M (decoding: one row per sequence),
// bfloat16 operands, float32 accumulation on the tensor cores (mma.sync m16n8k16).
//
// With few rows the product is bound by reading W once, and for the small matrices of a
// decoder layer by memory latency: the whole matrix has to be in flight at once.  The roles
// are therefore swapped (16 rows of W are the M side of the MMA, 8 rows of A its N side), and
// a CTA of eight warps owns 16 rows of W over a range of K: the warps take the 32-wide k steps
// of that range in turn, each issuing the 16-byte loads of four steps (straight into MMA
// fragments, the k index inside a step permuted identically for both operands) before it
// uses any of them.  A is small and is read through L1/L2.  The warps' partial sums are added
// in shared memory in the order of the warps.
//
// For matrices with few rows K is also cut into `splits` ranges over several CTAs; each
// writes its sums to scratch, and the CTA that finishes last for its 16 rows adds them in the
// order of the ranges and applies the epilogue.  `splits` depends on N and K only, so a row's
// result does not depend on how many rows are beside it.
//
// pico-engine leaves decode products to float32 cuBLAS (src/pico_engine/model.py:148-150, 177,
// 213, 223, 235) or its quantized Triton GEMVs (src/pico_engine/kernels.py:161-344).
#include "common.cuh"

#define LM_WARPS 8
#define LM_ROWS 16                     // rows of W per CTA
#define LM_UNROLL 4                    // k steps whose loads a warp has in flight
#define LM_MAX_M 64
#define LM_MAX_SPLITS 16

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Activations were written by the preceding kernel: a plain (coherent) load, never the read-only path.
__device__ __forceinline__ uint4 ld_act(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// epilogue: 0 store float32, 1 store bfloat16, 2 add into float32
__device__ __forceinline__ void lm_store(void* out, int epilogue, size_t o, float v) {
    if (epilogue == 0) ((float*)out)[o] = v;
    else if (epilogue == 1) ((bf16*)out)[o] = __float2bfloat16_rn(v);
    else ((float*)out)[o] += v;
}

// NT: number of 8-row tiles of A (M <= 8 * NT)
template <int NT>
__global__ void __launch_bounds__(32 * LM_WARPS) linear_mma_kernel(
    const bf16* A, const bf16* W, const void* bias, int bias_dtype,
    void* out, int epilogue, int M, int N, int K, int splits, int k_per_split,
    float* partial, unsigned int* tickets) {
    __shared__ float red[LM_WARPS][NT * 4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * LM_ROWS;
    const int split = blockIdx.y;
    const int k_begin = split * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const int n_steps = (k_end - k_begin + 31) / 32;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }

    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool ok0 = r0 < N, ok1 = r1 < N;
    const bf16* w0 = W + (size_t)(ok0 ? r0 : 0) * K;
    const bf16* w1 = W + (size_t)(ok1 ? r1 : 0) * K;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    pdl_launch_dependents();
    bool waited = false;
    for (int base = warp; base < n_steps; base += LM_WARPS * LM_UNROLL) {
        uint4 wa[LM_UNROLL], wb[LM_UNROLL];
#pragma unroll
        for (int u = 0; u < LM_UNROLL; ++u) {              // all loads of W first: they are what the kernel waits for
            const int k = k_begin + (base + u * LM_WARPS) * 32 + t * 8;
            const bool kin = k < k_end;                    // K and k_per_split are multiples of 8
            wa[u] = (ok0 && kin) ? ldg_stream(w0 + k) : zero;
            wb[u] = (ok1 && kin) ? ldg_stream(w1 + k) : zero;
        }
        if (!waited) { pdl_wait(); waited = true; }        // W is never written by a kernel; A is the predecessor's output
#pragma unroll
        for (int u = 0; u < LM_UNROLL; ++u) {
            const int k = k_begin + (base + u * LM_WARPS) * 32 + t * 8;
            const bool kin = k < k_end;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int m = j * 8 + g;
                const uint4 a = (m < M && kin) ? ld_act(A + (size_t)m * K + k) : zero;
                mma_bf16(acc[j], wa[u].x, wb[u].x, wa[u].y, wb[u].y, a.x, a.y);
                mma_bf16(acc[j], wa[u].z, wb[u].z, wa[u].w, wb[u].w, a.z, a.w);
            }
        }
    }
    if (!waited) pdl_wait();

    // acc[j][e] of lane (g, t): W row n0 + g + (e & 2 ? 8 : 0), A row j*8 + 2t + (e & 1)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][j * 4 + e][lane] = acc[j][e];
    __syncthreads();
    for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += 32 * LM_WARPS) {
        const int je = idx >> 5, ln = idx & 31;
        const int n = n0 + (ln >> 2) + ((je & 2) ? 8 : 0), m = (je >> 2) * 8 + 2 * (ln & 3) + (je & 1);
        if (n >= N || m >= M) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < LM_WARPS; ++w) v += red[w][je][ln];
        if (splits == 1) {
            if (bias) v += load_as_f(bias, bias_dtype, n);
            lm_store(out, epilogue, (size_t)m * N + n, v);
        } else {
            partial[((size_t)split * M + m) * N + n] = v;
        }
    }
    if (splits == 1) return;

    __shared__ unsigned int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&tickets[blockIdx.x], 1u);
        s_last = (prev == (unsigned int)splits - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int rows = min(LM_ROWS, N - n0);
    for (int idx = threadIdx.x; idx < rows * M; idx += blockDim.x) {
        const int m = idx / rows, n = n0 + idx % rows;
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += __ldcg(&partial[((size_t)s * M + m) * N + n]);
        if (bias) v += load_as_f(bias, bias_dtype, n);
        lm_store(out, epilogue, (size_t)m * N + n, v);
    }
    if (threadIdx.x == 0) tickets[blockIdx.x] = 0u;          // ready for the next launch
}

// The number of K ranges for an [N, K] weight: about two CTAs per SM for matrices with few
// rows, at least 256 columns each.  A function of N and K only.
extern "C" int pe_linear_mma_splits(int N, int K) {
    const int tiles = (N + LM_ROWS - 1) / LM_ROWS;
    int s = (2 * 148 + tiles - 1) / tiles;
    if (s > K / 256) s = K / 256;
    if (s > LM_MAX_SPLITS) s = LM_MAX_SPLITS;
    return s < 1 ? 1 : s;
}

extern "C" long long pe_linear_mma_scratch_bytes(int M, int N, int K) {
    const int s = pe_linear_mma_splits(N, K);
    return s > 1 ? (long long)s * M * N * 4 : 0;
}

// `tickets` holds at least ceil(N / 16) zeroed unsigned ints; the kernel leaves them zero.
extern "C" int pe_linear_mma(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                             int M, int N, int K, void* partial, void* tickets, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > LM_MAX_M || K <= 0 || K % 8 || epilogue < 0 || epilogue > 2) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return PE_ERR_UNSUPPORTED;
    const int splits = pe_linear_mma_splits(N, K);
    if (splits > 1 && (!partial || !tickets)) return PE_ERR_UNSUPPORTED;
    int k_per_split = (K + splits - 1) / splits;
    k_per_split = (k_per_split + 31) / 32 * 32;
    dim3 grid((N + LM_ROWS - 1) / LM_ROWS, splits);
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = (M + 7) / 8;
#define LM_GO(NT) PE_TRY(pe_launch(linear_mma_kernel<NT>, grid, 32 * LM_WARPS, 0, s, (const bf16*)A, (const bf16*)W, bias, bias_dtype, out, \
        epilogue, M, N, K, splits, k_per_split, (float*)partial, (unsigned int*)tickets))
    switch (nt) {
        case 1: LM_GO(1); break;
        case 2: LM_GO(2); break;
        case 3: LM_GO(3); break;
        case 4: LM_GO(4); break;
        case 5: LM_GO(5); break;
        case 6: LM_GO(6); break;
        case 7: LM_GO(7); break;
        default: LM_GO(8); break;
    }
#undef LM_GO
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- the same product without any allocation
// See linear_mma_static.h.  The scratch of the split ranges lives in this file-scope device
// array.  Its name is a device symbol: host code may not pass `static_scratch` itself to a
// kernel (on the host it is only a stand-in for the symbol), so the device address is looked
// up once per device with cudaGetSymbolAddress and that pointer is what the kernel gets.
#include "linear_mma_static.h"
#include <mutex>

static __device__ __align__(256) unsigned char static_scratch[PE_STATIC_SCRATCH_BYTES + PE_STATIC_TICKETS * sizeof(unsigned int)];

#define PE_STATIC_MAX_DEVICES 64
static void* static_scratch_address[PE_STATIC_MAX_DEVICES];     // device address of static_scratch, per device
static std::mutex static_scratch_mutex;

// The device address of the array on the current device; looked up on the first call there.
static int static_scratch_on_current_device(void** address) {
    int device = -1;
    PE_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= PE_STATIC_MAX_DEVICES) return PE_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(static_scratch_mutex);
    if (!static_scratch_address[device]) {
        void* p = nullptr;
        PE_TRY(cudaGetSymbolAddress(&p, static_scratch));       // with `device` current: its copy of the array
        static_scratch_address[device] = p;
    }
    *address = static_scratch_address[device];
    return 0;
}

extern "C" int pe_linear_mma_static(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                                    int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > LM_MAX_M || K <= 0 || K % 8 || epilogue < 0 || epilogue > 2) return PE_ERR_UNSUPPORTED;
    const int splits = pe_linear_mma_splits(N, K);
    const long long partial_bytes = pe_linear_mma_scratch_bytes(M, N, K);
    const long long tickets = splits > 1 ? (N + LM_ROWS - 1) / LM_ROWS : 0;
    if (partial_bytes > (long long)PE_STATIC_SCRATCH_BYTES || tickets > (long long)PE_STATIC_TICKETS)
        return PE_ERR_STATIC_TOO_LARGE;
    void* base = nullptr;
    const int rc = static_scratch_on_current_device(&base);
    if (rc) return rc;
    unsigned char* ticket_area = (unsigned char*)base + PE_STATIC_SCRATCH_BYTES;
    if (tickets)                                                 // whatever an earlier call left: tickets start at zero
        PE_TRY(cudaMemsetAsync(ticket_area, 0, (size_t)tickets * sizeof(unsigned int), (cudaStream_t)stream));
    return pe_linear_mma(A, W, bias, bias_dtype, out, epilogue, M, N, K, base, ticket_area, stream);
}
