// out = A[M, K] . W[N, K]^T for many rows (prompts), bfloat16 operands, on the 5th-generation
// tensor cores: tcgen05.mma with both operands in shared memory and the float32 accumulator
// in tensor memory, fused with what follows the product in a decoder layer.
//
//   one CTA = one 128 x BN tile of the output (BN = 128, or 256 = 128 gate + 128 up columns)
//   warp 0     producer: TMA tiled loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a
//              128 x 64 tile of A and a BN x 64 tile of W per k block into a ring of stages
//   warp 1     allocates tensor memory; one lane issues four tcgen05.mma (K = 16 each) per
//              stage and commits them to the stage's "empty" barrier, the last to "accumulator full"
//   warps 2-5  epilogue: tcgen05.ld of 32 columns at a time (lane = output row), then
//                STORE   out[M, N] = acc + bias, bfloat16               (q/k/v projection)
//                ACCUM   x[M, N] += acc, float32                        (o-proj, down-proj: the residual sum)
//                SWIGLU  act[M, I] = silu(acc[:, c]) * acc[:, 128 + c]  (gate/up; W tile = rows n0.. and I + n0..)
//
// Every mbarrier wait is bounded by the clock; a wait that runs out sets *status to 2, the
// roles leave their loops, tensor memory is freed and the CTA returns.
//
// pico-engine leaves these products to cuBLAS under fp16 autocast and runs bias, residual and
// activation as parts of, or beside, those library calls (src/pico_engine/model.py:177, 213, 223-235).
#include "common.cuh"
#include <cuda.h>

#define GT_BM 128
#define GT_BK 64
#define GT_STAGES 4
#define GT_THREADS 192
#define GT_WAIT_CYCLES 2000000000ll

enum { GT_STORE = 0, GT_ACCUM = 1, GT_SWIGLU = 2 };

struct GtArgs {
    void* out; const void* bias; int bias_dtype;
    int M, N, K;           // N: rows of W that make output columns (SWIGLU: N = 2 I)
    int I;                 // SWIGLU: columns of the result
};

__device__ __forceinline__ unsigned gt_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool gt_wait(unsigned bar, unsigned parity) {
    const long long deadline = clock64() + GT_WAIT_CYCLES;
    for (;;) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() > deadline) return false;
    }
}
__device__ __forceinline__ void gt_tma_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// K-major operand tile [rows][64 bfloat16] in 128-byte swizzle: 8-row groups are 1024 bytes apart
__device__ __forceinline__ unsigned long long gt_desc(unsigned smem_addr) {
    return (unsigned long long)((smem_addr >> 4) & 0x3FFFu) | ((unsigned long long)(1024u >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void gt_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void gt_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gt_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ unsigned gt_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GT_THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  const GtArgs p, int* status) {
    extern __shared__ __align__(1024) unsigned char gt_mem[];       // [stage][A tile 16 KB | W tile BN * 128 B]
    __shared__ __align__(8) unsigned long long full_bar[GT_STAGES], empty_bar[GT_STAGES], acc_bar;
    __shared__ unsigned tmem_base_s;
    constexpr unsigned A_BYTES = GT_BM * GT_BK * 2, W_BYTES = BN * GT_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * GT_BM;
    const int n0 = blockIdx.y * (EPI == GT_SWIGLU ? 128 : BN);     // SWIGLU: 128 result columns per CTA
    const int k_blocks = (p.K + GT_BK - 1) / GT_BK;
    // shared memory for the stages, 1024-byte aligned as the swizzle needs
    const unsigned stage0 = (gt_smem(gt_mem) + 1023u) & ~1023u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GT_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&full_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&empty_bar[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&acc_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                                // tensor memory: BN columns of 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"((unsigned)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_base_s;
    // Only now may the next kernel of the stream be scheduled: if it came earlier, took tensor memory on this SM
    // and then waited for this grid to end, a CTA of this grid that still had to allocate would wait for it in turn.
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {                                            // ---------------- producer
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % GT_STAGES;
                if (kb >= GT_STAGES && !gt_wait(gt_smem(&empty_bar[s]), (unsigned)((kb / GT_STAGES) - 1) & 1u)) { atomicExch(status, 2); break; }
                const unsigned bar = gt_smem(&full_bar[s]), dst = stage0 + s * STAGE_BYTES;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STAGE_BYTES) : "memory");
                gt_tma_2d(dst, &map_a, kb * GT_BK, m0, bar);
                if (EPI == GT_SWIGLU) {
                    gt_tma_2d(dst + A_BYTES, &map_w, kb * GT_BK, n0, bar);                       // gate rows
                    gt_tma_2d(dst + A_BYTES + W_BYTES / 2, &map_w, kb * GT_BK, p.I + n0, bar);   // the matching up rows
                } else {
                    gt_tma_2d(dst + A_BYTES, &map_w, kb * GT_BK, n0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                            // ---------------- MMA issuer
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = BN, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(GT_BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % GT_STAGES;
                if (!gt_wait(gt_smem(&full_bar[s]), (unsigned)(kb / GT_STAGES) & 1u)) { atomicExch(status, 2); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long da = gt_desc(stage0 + s * STAGE_BYTES), dw = gt_desc(stage0 + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                for (int kk = 0; kk < GT_BK / 16; ++kk)              // 16 columns = 32 bytes further inside the swizzle atom
                    gt_mma(tmem, da + 2ull * kk, dw + 2ull * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                gt_commit(gt_smem(&empty_bar[s]));                   // the stage is free once these MMAs have read it
            }
            gt_commit(gt_smem(&acc_bar));                            // all MMAs done: the accumulator is complete
        }
    } else {                                                        // ---------------- epilogue, warps 2..5
        const int quarter = warp & 3;                               // the 32 lanes of tensor memory this warp may read
        const int row = m0 + quarter * 32 + lane;
        if (gt_wait(gt_smem(&acc_bar), 0u)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16);
            if (EPI == GT_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    float gate[32], up[32];
                    gt_ld32(taddr + c, gate);
                    gt_ld32(taddr + 128 + c, up);
                    if (row < p.M) {
                        bf16* o = (bf16*)p.out + (size_t)row * p.I + n0 + c;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (n0 + c + i < p.I) {                 // I is a multiple of 8
                                unsigned w[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    // gate and up are rounded to bfloat16 first, as the unfused path stores them
                                    const float g0 = __bfloat162float(__float2bfloat16_rn(gate[i + 2 * e])), g1 = __bfloat162float(__float2bfloat16_rn(gate[i + 2 * e + 1]));
                                    const float u0 = __bfloat162float(__float2bfloat16_rn(up[i + 2 * e])), u1 = __bfloat162float(__float2bfloat16_rn(up[i + 2 * e + 1]));
                                    w[e] = gt_pack(g0 * (1.0f / (1.0f + expf(-g0))) * u0, g1 * (1.0f / (1.0f + expf(-g1))) * u1);
                                }
                                *reinterpret_cast<uint4*>(o + i) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    float acc[32];
                    gt_ld32(taddr + c, acc);
                    if (row < p.M && n0 + c < p.N) {
                        if (EPI == GT_STORE) {
                            bf16* o = (bf16*)p.out + (size_t)row * p.N + n0 + c;
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                if (n0 + c + i < p.N) {             // N is a multiple of 8
                                    unsigned w[4];
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        float a = acc[i + 2 * e], b = acc[i + 2 * e + 1];
                                        if (p.bias) { a += load_as_f(p.bias, p.bias_dtype, n0 + c + i + 2 * e); b += load_as_f(p.bias, p.bias_dtype, n0 + c + i + 2 * e + 1); }
                                        w[e] = gt_pack(a, b);
                                    }
                                    *reinterpret_cast<uint4*>(o + i) = make_uint4(w[0], w[1], w[2], w[3]);
                                }
                            }
                        }
                    }
                    if (EPI == GT_ACCUM) {
                        // Into the float32 residual stream (the sum stays float32, as in the decode kernels).  A lane
                        // holds a row, so the warp turns its 32 x 32 block through shared memory (the stages are free:
                        // every MMA has read them) and then adds row by row, 32 lanes to 128 contiguous bytes.
                        float* turn = reinterpret_cast<float*>(gt_mem + (stage0 - gt_smem(gt_mem))) + quarter * (32 * 33);
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 32; ++i) turn[lane * 33 + i] = acc[i];
                        __syncwarp();
                        const int col = n0 + c + lane;
                        if (col < p.N) {
                            float* o = (float*)p.out + (size_t)(m0 + quarter * 32) * p.N + col;
                            const int rows = min(32, p.M - (m0 + quarter * 32));
                            float x[32];                             // all loads first: they do not wait for one another
#pragma unroll
                            for (int r = 0; r < 32; ++r) x[r] = r < rows ? o[(size_t)r * p.N] : 0.f;
#pragma unroll
                            for (int r = 0; r < 32; ++r) if (r < rows) o[(size_t)r * p.N] = x[r] + turn[r * 33 + lane];
                        }
                    }
                }
            }
        } else {
            atomicExch(status, 2);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)BN) : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*gt_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static gt_encode_fn gt_encoder() {
    static gt_encode_fn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (gt_encode_fn)sym;
    }
    return fn;
}

// a [rows, K] bfloat16 row-major matrix, loaded in boxes of 64 columns x box_rows rows with 128-byte swizzle
static int gt_make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
    gt_encode_fn enc = gt_encoder();
    if (!enc) return PE_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {GT_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

template <int BN, int EPI>
static int gt_launch(const CUtensorMap& ma, const CUtensorMap& mw, const GtArgs& p, dim3 grid, int* status, cudaStream_t s) {
    const size_t smem = (size_t)GT_STAGES * (GT_BM * GT_BK * 2 + BN * GT_BK * 2) + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        PE_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    PE_TRY(pe_launch(gemm_tcgen05_kernel<BN, EPI>, grid, GT_THREADS, smem, s, ma, mw, p, status));
    return 0;
}

// epilogue 0: out bfloat16 [M, N] = A . W^T + bias;  1: float32 out [M, N] += A . W^T;
//          2: out bfloat16 [M, N / 2] = silu(A . Wg^T) * (A . Wu^T), W = [Wg; Wu]
extern "C" int pe_gemm_tcgen05(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                               int M, int N, int K, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || N % 8 || epilogue < 0 || epilogue > 2 || !status) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)out) & 15) return PE_ERR_UNSUPPORTED;
    if (epilogue == 2 && (N % 16 || bias)) return PE_ERR_UNSUPPORTED;
    CUtensorMap ma, mw;
    int rc = gt_make_map(&ma, A, M, K, GT_BM);
    if (rc) return rc;
    rc = gt_make_map(&mw, W, N, K, 128);
    if (rc) return rc;
    GtArgs p = {};
    p.out = out; p.bias = bias; p.bias_dtype = bias_dtype; p.M = M; p.N = N; p.K = K; p.I = N / 2;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned mt = (M + GT_BM - 1) / GT_BM;
    if (epilogue == 2) return gt_launch<256, GT_SWIGLU>(ma, mw, p, dim3(mt, (N / 2 + 127) / 128), status, s);
    if (epilogue == 0) return gt_launch<128, GT_STORE>(ma, mw, p, dim3(mt, (N + 127) / 128), status, s);
    return gt_launch<128, GT_ACCUM>(ma, mw, p, dim3(mt, (N + 127) / 128), status, s);
}
