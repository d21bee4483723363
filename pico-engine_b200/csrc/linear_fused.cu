// The matrix products of a decode step for up to 16 rows (sequences), each fused with what
// stands before and after it in the layer, so that a layer is five kernels instead of ten:
//
//   prologue  PLAIN     A is bfloat16 [M, K]
//             RMSNORM   A = bfloat16(x * rsqrt(mean(x^2) + eps) * w) from the float32 residual stream x
//   epilogue  STORE     out[M, N] = acc (+ bias), bfloat16 or float32
//             ACCUM     x[M, N] += acc (+ bias) in float32 (the residual sum)
//             SWIGLU    out[M, I] = silu(gate) * up, gate and up being rows i and I + i of W
//             ROPE      rows are query, key and value heads: add bias, rotate query and key heads
//                       by position, write queries to out and keys and values into the paged cache
//
// At these sizes a product is bound by memory latency, not bandwidth: what counts is the number
// of dependent trips to memory.  A CTA of eight warps owns 8 or 16 rows of W over all of K (no
// split over CTAs, hence no second pass), its warps take the 32-wide k steps in turn, and every
// warp issues the loads of four steps of W before it waits for the preceding kernel
// (griddepcontrol.wait) and touches activations.  The roles of the MMA operands are swapped as
// in linear_mma.cu: rows of W are the M side of mma.sync m16n8k16, sequences the N side.  The
// 16 rows of a tile are two groups of 8: for SWIGLU the matching gate and up rows, for ROPE
// the two halves of a head that rotate together, so the epilogue finds its pairs in one CTA.
//
// pico-engine runs these as separate launches: rmsnorm, F.linear, rope, index_copy_, addmm,
// silu_mul (src/pico_engine/model.py:175-235).
#include "common.cuh"

#define LF_WARPS 8
#define LF_UNROLL 4

enum { LF_PLAIN = 0, LF_RMSNORM = 1 };
enum { LF_STORE_F32 = 0, LF_STORE_BF16 = 1, LF_ACCUM = 2, LF_SWIGLU = 3, LF_ROPE = 4 };

struct LfArgs {
    // operands
    const bf16* A;            // PLAIN: [M, K]
    const float* X;           // RMSNORM: [M, K]
    const void* norm_w; int norm_w_dtype; float eps;
    const bf16* W;            // [N, K]
    const void* bias; int bias_dtype;
    void* out;                // STORE: [M, N]; ACCUM: float [M, N]; SWIGLU: bf16 [M, I]; ROPE: bf16 [M, n_q * hd]
    int M, N, K;
    int rows;                 // STORE/ACCUM: rows of W per CTA, 8 or 16
    int I;                    // SWIGLU
    // ROPE
    int n_q, n_kv, hd;
    const float* cos_t; const float* sin_t;
    const int* tok_pos; const int* tok_row;
    bf16* k_pool; bf16* v_pool; const int* block_table; int table_stride; int store;
};

__device__ __forceinline__ uint4 lf_ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lf_ld16(const void* p) {       // coherent: data of the preceding kernel
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void lf_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned lf_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// NT: 8-row tiles of sequences (M <= 8 * NT)
template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(32 * LF_WARPS) linear_fused_kernel(const LfArgs p) {
    __shared__ float red[LF_WARPS][NT * 4][32];
    __shared__ float ssq[LF_WARPS][NT * 8];
    __shared__ float rstd_s[NT * 8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int K = p.K, M = p.M;

    // which rows of W this lane streams: r_lo feeds MMA rows 0-7, r_hi rows 8-15
    int r_lo, r_hi;
    if (EPI == LF_SWIGLU) {
        r_lo = blockIdx.x * 8 + g; r_hi = p.I + r_lo;
    } else if (EPI == LF_ROPE) {
        const int half = p.hd >> 1, per_head = half >> 3;
        r_lo = (blockIdx.x / per_head) * p.hd + (blockIdx.x % per_head) * 8 + g; r_hi = r_lo + half;
    } else {
        r_lo = blockIdx.x * p.rows + g; r_hi = p.rows == 16 ? r_lo + 8 : p.N;
    }
    const bool ok_lo = r_lo < p.N, ok_hi = r_hi < p.N;
    const bf16* w_lo = p.W + (size_t)(ok_lo ? r_lo : 0) * K;
    const bf16* w_hi = p.W + (size_t)(ok_hi ? r_hi : 0) * K;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int n_steps = (K + 31) / 32;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    pdl_launch_dependents();
    uint4 wa[LF_UNROLL], wb[LF_UNROLL];
#pragma unroll
    for (int u = 0; u < LF_UNROLL; ++u) {                   // W first: no kernel writes it, so it need not wait
        const int k = (warp + u * LF_WARPS) * 32 + t * 8;
        wa[u] = (ok_lo && k < K) ? lf_ldg_stream(w_lo + k) : zero;
        wb[u] = (ok_hi && k < K) ? lf_ldg_stream(w_hi + k) : zero;
    }
    pdl_wait();                                             // from here on the preceding kernel's results may be read
    if (PRO == LF_RMSNORM) {
        // sum of squares of every row of x: each warp over the k steps it owns, then over the warps
        float part[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) part[j] = 0.f;
        for (int b2 = warp; b2 < n_steps; b2 += LF_WARPS) {
            const int k = b2 * 32 + t * 8;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int m = j * 8 + g;
                if (m < M && k < K) {
                    const float4 x0 = *reinterpret_cast<const float4*>(p.X + (size_t)m * K + k);
                    const float4 x1 = *reinterpret_cast<const float4*>(p.X + (size_t)m * K + k + 4);
                    part[j] += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w +
                               x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            part[j] += __shfl_xor_sync(0xffffffffu, part[j], 1);
            part[j] += __shfl_xor_sync(0xffffffffu, part[j], 2);
            if (t == 0) ssq[warp][j * 8 + g] = part[j];
        }
        __syncthreads();
        if (threadIdx.x < NT * 8) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < LF_WARPS; ++w) sum += ssq[w][threadIdx.x];
            rstd_s[threadIdx.x] = 1.0f / sqrtf(sum / (float)K + p.eps);
        }
        __syncthreads();
    }
    for (int base = warp; base < n_steps; base += LF_WARPS * LF_UNROLL) {
        if (base != warp) {
#pragma unroll
            for (int u = 0; u < LF_UNROLL; ++u) {
                const int k = (base + u * LF_WARPS) * 32 + t * 8;
                wa[u] = (ok_lo && k < K) ? lf_ldg_stream(w_lo + k) : zero;
                wb[u] = (ok_hi && k < K) ? lf_ldg_stream(w_hi + k) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < LF_UNROLL; ++u) {
            const int k = (base + u * LF_WARPS) * 32 + t * 8;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int m = j * 8 + g;
                uint4 a = zero;
                if (m < M && k < K) {
                    if (PRO == LF_RMSNORM) {
                        const float4 x0 = *reinterpret_cast<const float4*>(p.X + (size_t)m * K + k);
                        const float4 x1 = *reinterpret_cast<const float4*>(p.X + (size_t)m * K + k + 4);
                        const float r = rstd_s[m];
                        a.x = lf_pack(x0.x * r * load_as_f(p.norm_w, p.norm_w_dtype, k), x0.y * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 1));
                        a.y = lf_pack(x0.z * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 2), x0.w * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 3));
                        a.z = lf_pack(x1.x * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 4), x1.y * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 5));
                        a.w = lf_pack(x1.z * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 6), x1.w * r * load_as_f(p.norm_w, p.norm_w_dtype, k + 7));
                    } else {
                        a = lf_ld16(p.A + (size_t)m * K + k);
                    }
                }
                lf_mma(acc[j], wa[u].x, wb[u].x, wa[u].y, wb[u].y, a.x, a.y);
                lf_mma(acc[j], wa[u].z, wb[u].z, wa[u].w, wb[u].w, a.z, a.w);
            }
        }
    }

    // acc[j][e] of lane (g, t): MMA row g (+8 if e & 2), sequence j*8 + 2t + (e & 1)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][j * 4 + e][lane] = acc[j][e];
    __syncthreads();

    // one thread per (sequence, row of the tile's first group); it sums both groups over the warps
    for (int idx = threadIdx.x; idx < NT * 64; idx += 32 * LF_WARPS) {
        const int j = idx >> 6, e1 = (idx >> 5) & 1, ln = idx & 31;
        const int r = ln >> 2, m = j * 8 + 2 * (ln & 3) + e1;
        if (m >= M) continue;
        float v_lo = 0.f, v_hi = 0.f;
#pragma unroll
        for (int w = 0; w < LF_WARPS; ++w) { v_lo += red[w][j * 4 + e1][ln]; v_hi += red[w][j * 4 + 2 + e1][ln]; }

        if (EPI == LF_SWIGLU) {
            const int i = blockIdx.x * 8 + r;
            if (i < p.I) {
                // the unfused path rounds gate and up to bfloat16 before the activation; so does this one
                v_lo = __bfloat162float(__float2bfloat16_rn(v_lo)); v_hi = __bfloat162float(__float2bfloat16_rn(v_hi));
                const float sig = 1.0f / (1.0f + expf(-v_lo));
                ((bf16*)p.out)[(size_t)m * p.I + i] = __float2bfloat16_rn(v_lo * sig * v_hi);
            }
        } else if (EPI == LF_ROPE) {
            const int half = p.hd >> 1, per_head = half >> 3;
            const int head = blockIdx.x / per_head, d = (blockIdx.x % per_head) * 8 + r;   // d < half
            const int n_lo = head * p.hd + d, n_hi = n_lo + half;
            if (p.bias) { v_lo += load_as_f(p.bias, p.bias_dtype, n_lo); v_hi += load_as_f(p.bias, p.bias_dtype, n_hi); }
            // the unfused path rounds the projection to bfloat16 before it rotates; so does this one
            v_lo = __bfloat162float(__float2bfloat16_rn(v_lo)); v_hi = __bfloat162float(__float2bfloat16_rn(v_hi));
            const int pos = p.tok_pos[m];
            if (head < p.n_q + p.n_kv && p.cos_t) {
                const float c = p.cos_t[(size_t)pos * half + d], s = p.sin_t[(size_t)pos * half + d];
                const float a = v_lo * c - v_hi * s, b = v_lo * s + v_hi * c;
                v_lo = a; v_hi = b;
            }
            const bf16 o_lo = __float2bfloat16_rn(v_lo), o_hi = __float2bfloat16_rn(v_hi);
            if (head < p.n_q) {
                bf16* q = (bf16*)p.out + (size_t)m * p.n_q * p.hd + (size_t)head * p.hd;
                q[d] = o_lo; q[d + half] = o_hi;
            } else if (p.store) {
                const int page = p.block_table[(size_t)p.tok_row[m] * p.table_stride + pos / PE_PAGE];
                if (page >= 0) {
                    const bool is_k = head < p.n_q + p.n_kv;
                    const int kvh = head - p.n_q - (is_k ? 0 : p.n_kv);
                    bf16* dst = (is_k ? p.k_pool : p.v_pool) +
                                (((size_t)page * p.n_kv + kvh) * PE_PAGE + (pos % PE_PAGE)) * p.hd;
                    dst[d] = o_lo; dst[d + half] = o_hi;
                }
            }
        } else {
            const int n_lo = blockIdx.x * p.rows + r, n_hi = n_lo + 8;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int n = h ? n_hi : n_lo;
                if (n >= p.N || (h && p.rows != 16)) continue;
                float v = h ? v_hi : v_lo;
                if (p.bias) v += load_as_f(p.bias, p.bias_dtype, n);
                const size_t o = (size_t)m * p.N + n;
                if (EPI == LF_STORE_F32) ((float*)p.out)[o] = v;
                else if (EPI == LF_STORE_BF16) ((bf16*)p.out)[o] = __float2bfloat16_rn(v);
                else ((float*)p.out)[o] += v;
            }
        }
    }
}

template <int PRO, int EPI>
static int lf_launch(const LfArgs& a, int tiles, cudaStream_t s) {
    if (a.M <= 8) PE_TRY(pe_launch(linear_fused_kernel<1, PRO, EPI>, tiles, 32 * LF_WARPS, 0, s, a));
    else PE_TRY(pe_launch(linear_fused_kernel<2, PRO, EPI>, tiles, 32 * LF_WARPS, 0, s, a));
    return 0;
}

static bool lf_aligned(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// x += a . W^T (+ bias) or out = a . W^T (+ bias); `a` bfloat16 [M <= 16, K], or with `x_norm`
// the float32 rows whose RMSNorm (weights norm_w, eps) is the operand.
// epilogue: 0 store float32, 1 store bfloat16, 2 add into float32 out.
extern "C" int pe_linear_fused(const void* a, const float* x_norm, const void* norm_w, int norm_w_dtype, float eps,
                               const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M, int N,
                               int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 || epilogue < 0 || epilogue > 2 || !lf_aligned(W) || !lf_aligned(x_norm ? (const void*)x_norm : a))
        return PE_ERR_UNSUPPORTED;
    LfArgs p = {};
    p.A = (const bf16*)a; p.X = x_norm; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps;
    p.W = (const bf16*)W; p.bias = bias; p.bias_dtype = bias_dtype; p.out = out; p.M = M; p.N = N; p.K = K;
    p.rows = (N + 15) / 16 >= 2 * 148 ? 16 : 8;              // small matrices: more, thinner CTAs
    const int tiles = (N + p.rows - 1) / p.rows;
    cudaStream_t s = (cudaStream_t)stream;
    if (x_norm) {
        if (epilogue == 0) return lf_launch<LF_RMSNORM, LF_STORE_F32>(p, tiles, s);
        if (epilogue == 1) return lf_launch<LF_RMSNORM, LF_STORE_BF16>(p, tiles, s);
        return lf_launch<LF_RMSNORM, LF_ACCUM>(p, tiles, s);
    }
    if (epilogue == 0) return lf_launch<LF_PLAIN, LF_STORE_F32>(p, tiles, s);
    if (epilogue == 1) return lf_launch<LF_PLAIN, LF_STORE_BF16>(p, tiles, s);
    return lf_launch<LF_PLAIN, LF_ACCUM>(p, tiles, s);
}

// act[M, I] = silu(h . Wg^T) * (h . Wu^T), h = RMSNorm(x); W = [Wg; Wu] is [2I, K].
extern "C" int pe_norm_gate_up_swiglu(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* W,
                                      void* act, int M, int I, int K, void* stream) {
    if (M <= 0 || I <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 || I % 8 || !lf_aligned(W) || !lf_aligned(x)) return PE_ERR_UNSUPPORTED;
    LfArgs p = {};
    p.X = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps; p.W = (const bf16*)W; p.out = act;
    p.M = M; p.N = 2 * I; p.K = K; p.I = I; p.rows = 16;
    return lf_launch<LF_RMSNORM, LF_SWIGLU>(p, I / 8, (cudaStream_t)stream);
}

// q[M, n_q * hd] and the cache pages of keys and values from h = RMSNorm(x) (or from bfloat16
// `a` when x is null): project with W = [Wq; Wk; Wv], add bias, rotate q and k by position
// (cos_t null: no rotation), write keys and values at (page of the token's sequence, position).
extern "C" int pe_norm_qkv_rope_store(const void* a, const float* x, const void* norm_w, int norm_w_dtype, float eps,
                                      const void* W, const void* bias, int bias_dtype, void* q_out, int M, int K,
                                      int n_q, int n_kv, int hd, const float* cos_t, const float* sin_t,
                                      const int* tok_pos, const int* tok_row, void* k_pool, void* v_pool,
                                      const int* block_table, int table_stride, int store, void* stream) {
    if (M <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 || hd % 16 || !lf_aligned(W) || !lf_aligned(x ? (const void*)x : a)) return PE_ERR_UNSUPPORTED;
    LfArgs p = {};
    p.A = (const bf16*)a; p.X = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps;
    p.W = (const bf16*)W; p.bias = bias; p.bias_dtype = bias_dtype; p.out = q_out; p.M = M; p.N = (n_q + 2 * n_kv) * hd;
    p.K = K; p.rows = 16; p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.cos_t = cos_t; p.sin_t = sin_t; p.tok_pos = tok_pos;
    p.tok_row = tok_row; p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.block_table = block_table;
    p.table_stride = table_stride; p.store = store;
    const int tiles = (n_q + 2 * n_kv) * (hd / 16);
    if (x) return lf_launch<LF_RMSNORM, LF_ROPE>(p, tiles, (cudaStream_t)stream);
    return lf_launch<LF_PLAIN, LF_ROPE>(p, tiles, (cudaStream_t)stream);
}
