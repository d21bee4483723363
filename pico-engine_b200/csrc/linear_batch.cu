// The matrix products of a decode step for 17 to 64 rows (sequences), each fused with what stands before and after it
// in the layer, as linear_fused.cu does for up to 16 rows:
//
//   prologue  PLAIN     A is bfloat16 [M, K]
//             RMSNORM   A = RMSNorm(x) of the float32 residual stream x: bfloat16(x * w) is multiplied and
//                       rsqrt(mean(x^2) + eps) applied to the sums, so x is read once
//   epilogue  STORE     out[M, N] = acc (+ bias), bfloat16
//             ACCUM     x[M, N] += acc (+ bias) in float32 (the residual sum), a reduction in memory
//             SWIGLU    out[M, I] = silu(gate) * up, gate and up being rows i and I + i of W
//             ROPE      rows are query, key and value heads: add bias, rotate query and key heads by position, write
//                       queries to out and keys and values into the paged cache
//
// With this many rows a 16-row tile of W a CTA (linear_fused.cu) would read the activations, which every CTA needs, four
// times as often as the weights; here a CTA owns 64 rows of W, so both cost the same and the products of a layer still
// have 100 to 150 CTAs: gate/up 152 tiles; the others (14 to 18 tiles of 64 rows) cut K into ranges, one CTA each, the
// CTAs of a tile a thread-block cluster whose partial sums go to the first CTA's shared memory (one bulk copy a CTA)
// and are added there in the order of the ranges.
//
//   warps 0-7   consumers: warp w multiplies rows 16 (w % 4) .. + 16 of the tile by tokens 32 (w / 4) .. + 32:
//               ldmatrix from shared memory, mma.sync m16n8k16 with rows of W as the M side and tokens as the N side
//   warps 8-11  producers: K in chunks of 128 columns through a ring of stages.  One thread issues TMA copies of boxes
//               of W (before griddepcontrol.wait: no kernel writes weights) and, PLAIN, of the activations: a few
//               copies a chunk (issuing a copy costs about 65 cycles, so one copy a row would take longer than the
//               chunk's arithmetic).  RMSNORM: the four warps read x as float32, scale it by the norm's weight, round
//               and store it in the layout the copies would have given, and sum the squares.
//
// Shared memory holds boxes of 64 columns (128 bytes a row) in the 128-byte swizzle of the copies: the 16-byte unit u of
// row r is stored at unit u ^ (r % 8), which also keeps ldmatrix free of bank conflicts.
//
// The 16 rows of a warp are two groups of 8 (MMA rows 0-7 and 8-15): for SWIGLU the matching gate and up rows, for
// ROPE the two halves of a head that rotate together, so a thread finds its pairs in its own registers.  The boxes are
// placed accordingly: [32 gate rows][32 up rows]; for ROPE, runs of 8, 16 or 32 rows (what divides half a head).
//
// Waiting on an mbarrier is bounded: a wait that runs out sets *status to 7, and the CTA goes on to its barriers without
// computing, so that no warp and no CTA of a cluster is left waiting.
//
// pico-engine runs these as separate launches: rmsnorm, F.linear, rope, index_copy_, addmm, silu_mul
// (src/pico_engine/model.py:175-235).
#include "common.cuh"
#include "tensor_map.cuh"

#define LB_TW 64                      // rows of W a CTA
#define LB_TM 64                      // tokens at most
#define LB_KC 128                     // columns of a chunk: two boxes of 64
#define LB_BOX (64 * 128)             // bytes of a box of 64 rows
#define LB_STAGE (4 * LB_BOX)         // W columns 0-63, W columns 64-127, tokens likewise
#define LB_CONSUMERS 8
#define LB_PRODUCERS 4
#define LB_THREADS (32 * (LB_CONSUMERS + LB_PRODUCERS))
#define LB_MAX_SPLIT 8
#define LB_MAX_STAGES 6
#define LB_WAIT_CYCLES 2000000000ll

enum { LB_PLAIN = 0, LB_RMSNORM = 1 };
enum { LB_STORE = 0, LB_ACCUM = 1, LB_SWIGLU = 2, LB_ROPE = 3 };

struct LbArgs {
    const float* X; const void* norm_w; int norm_w_dtype; float eps;
    const void* bias; int bias_dtype;
    void* out;
    int M, N, K;
    int stages, ksplit, chunks_per_split;
    int I;
    int n_q, n_kv, hd, run;           // run: rows of a box of W for ROPE (8, 16 or 32)
    const float* cos_t; const float* sin_t;
    const int* tok_pos; const int* tok_row;
    bf16* k_pool; bf16* v_pool; const int* block_table; int table_stride; int store;
};

__device__ __forceinline__ unsigned lb_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lb_bar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void lb_bar_expect(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lb_bar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool lb_bar_wait(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    const long long deadline = clock64() + LB_WAIT_CYCLES;
    for (;;) {
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() > deadline) return false;
    }
}
__device__ __forceinline__ void lb_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void lb_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ unsigned lb_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void lb_ldmatrix4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void lb_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned lb_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float lb_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Rows of a box of W, and the row of W at which box b (b * rows .. of the tile's 64 rows in shared memory) starts.
template <int EPI>
__device__ __forceinline__ int lb_box_rows(const LbArgs& p) { return EPI == LB_ROPE ? p.run : EPI == LB_SWIGLU ? 32 : 64; }
template <int EPI>
__device__ __forceinline__ int lb_box_first_row(const LbArgs& p, int tile, int b) {
    if (EPI == LB_SWIGLU) return tile * 32 + (b ? p.I : 0);                  // gate rows, then the matching up rows
    if (EPI == LB_ROPE) {                                                    // a run of pairs: dimensions d.., then d + hd / 2..
        const int half = p.hd >> 1, pi = tile * 32 + (b >> 1) * p.run, head = pi / half;
        return head * p.hd + (pi - head * half) + ((b & 1) ? half : 0);      // (past the last head: past N, and read as zeros)
    }
    return tile * LB_TW;
}
// The row of shared memory that holds row rr (0..15) of warp group rg: rows 0-7 the low group, 8-15 the high group.
template <int EPI>
__device__ __forceinline__ int lb_smem_row(const LbArgs& p, int rg, int rr) {
    if (EPI == LB_STORE || EPI == LB_ACCUM) return 16 * rg + rr;
    const int run = lb_box_rows<EPI>(p), pair = 8 * rg + (rr & 7);
    return (2 * (pair / run) + (rr >> 3)) * run + pair % run;
}

template <int PRO, int EPI, bool SPLIT>
__global__ void __launch_bounds__(LB_THREADS, 1) linear_batch_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_a, const LbArgs p, int* status) {
    extern __shared__ unsigned char lb_raw[];                    // [stage][W | W | tokens | tokens], then what the other ranges send
    __shared__ __align__(8) unsigned long long full_bar[LB_MAX_STAGES], empty_bar[LB_MAX_STAGES], gather_bar;
    __shared__ float ssq_tok[LB_TM];
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int ksplit = SPLIT ? p.ksplit : 1;
    const int tile = SPLIT ? blockIdx.x / ksplit : blockIdx.x, ks = SPLIT ? (int)lb_cluster_rank() : 0;
    const int n_chunks_all = (p.K + LB_KC - 1) / LB_KC;
    const int c_begin = ks * p.chunks_per_split, c_end = min(n_chunks_all, c_begin + p.chunks_per_split);
    const int n_chunks = max(0, c_end - c_begin), stages = p.stages, M = p.M;
    unsigned char* lb_mem = lb_raw + ((1024u - (lb_smem(lb_raw) & 1023u)) & 1023u);       // the swizzle wants boxes at multiples of 1024 bytes
    const unsigned mem0 = lb_smem(lb_mem), full0 = lb_smem(full_bar), empty0 = lb_smem(empty_bar), gbar = lb_smem(&gather_bar);
    float* gather = reinterpret_cast<float*>(lb_mem + (size_t)stages * LB_STAGE);      // [range - 1][64 x 64 sums | 64 sums of squares]
    constexpr int GATHER_FLOATS = LB_TW * LB_TM + LB_TM;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < stages; ++s) {
            lb_bar_init(full0 + 8u * s, PRO == LB_RMSNORM ? 1u + 32u * LB_PRODUCERS : 1u);
            lb_bar_init(empty0 + 8u * s, LB_CONSUMERS);
        }
        lb_bar_init(gbar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (SPLIT && ksplit > 1 && ks == 0) lb_bar_expect(gbar, (unsigned)((ksplit - 1) * GATHER_FLOATS * 4));
    }
    __syncthreads();
    if (SPLIT && ksplit > 1) lb_cluster_arrive();
    pdl_launch_dependents();

    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    bool ok = true;

    if (warp >= LB_CONSUMERS) {
        // ---------------------------------------------------------------- producers
        const int pt = threadIdx.x - 32 * LB_CONSUMERS, pw = pt >> 5, pl = pt & 31;
        auto issue_w = [&](int c) {                               // one thread
            const unsigned dst = mem0 + (c % stages) * LB_STAGE, bar = full0 + 8u * (c % stages);
            lb_bar_expect(bar, PRO == LB_PLAIN ? (unsigned)LB_STAGE : 2u * LB_BOX);
            const int x = (c_begin + c) * LB_KC, run = lb_box_rows<EPI>(p);
            for (int b = 0; b * run < LB_TW; ++b) {
                const int y = lb_box_first_row<EPI>(p, tile, b);
                pe_tma_load_2d(dst + b * run * 128, &map_w, x, y, bar);
                pe_tma_load_2d(dst + LB_BOX + b * run * 128, &map_w, x + 64, y, bar);
            }
        };
        auto issue_a = [&](int c) {                               // one thread, PLAIN
            const unsigned dst = mem0 + (c % stages) * LB_STAGE + 2 * LB_BOX, bar = full0 + 8u * (c % stages);
            const int x = (c_begin + c) * LB_KC;
            pe_tma_load_2d(dst, &map_a, x, 0, bar);
            pe_tma_load_2d(dst + LB_BOX, &map_a, x + 64, 0, bar);
        };
        const int ahead = min(n_chunks, stages);
        if (pt == 0)
            for (int c = 0; c < ahead; ++c) issue_w(c);           // weights: nothing to wait for
        pdl_wait();
        if (PRO == LB_PLAIN) {
            if (pt == 0) {
                for (int c = 0; c < ahead; ++c) issue_a(c);
                for (int c = ahead; c < n_chunks; ++c) {
                    if (!lb_bar_wait(empty0 + 8u * (c % stages), (unsigned)((c / stages) - 1) & 1u)) { ok = false; break; }
                    issue_w(c);
                    issue_a(c);
                }
            }
        } else {
            // RMSNORM: producer warp pw scales and rounds token rows pw, pw + 4, ...; its lane l columns 4 l .. 4 l + 3 of the
            // chunk (a row of the chunk is one coalesced load), and sums their squares.  Eight rows at a time, the next
            // eight loading meanwhile.
            float ssq[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) ssq[i] = 0.f;
            auto cols_of = [&](int c) { return min(LB_KC, p.K - (c_begin + c) * LB_KC); };
            auto load8 = [&](int c, int h, float4 (&x)[8]) {
                const size_t k0 = (size_t)(c_begin + c) * LB_KC + 4 * pl;
                const bool col_in = 4 * pl < cols_of(c);          // K is a multiple of 8: a group of 4 columns is inside or outside
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int tok = pw + 4 * (8 * h + i);
                    x[i] = (col_in && tok < M) ? *reinterpret_cast<const float4*>(p.X + (size_t)tok * p.K + k0) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
            auto load_w = [&](int c) {
                const size_t k0 = (size_t)(c_begin + c) * LB_KC + 4 * pl;
                if (4 * pl >= cols_of(c)) return make_float4(0.f, 0.f, 0.f, 0.f);
                if (p.norm_w_dtype == PE_BF16) {
                    const uint2 wv = *reinterpret_cast<const uint2*>((const bf16*)p.norm_w + k0);
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.y));
                    return make_float4(lo.x, lo.y, hi.x, hi.y);
                }
                return *reinterpret_cast<const float4*>((const float*)p.norm_w + k0);
            };
            // lane l's 8 bytes of token row r: box l / 16, unit (l % 16) / 2, swizzled by the row
            auto emit8 = [&](int c, int h, const float4 (&x)[8], const float4 w, float (&sq)[16]) {
                unsigned char* box = lb_mem + (size_t)(c % stages) * LB_STAGE + (2 + (pl >> 4)) * LB_BOX;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = pw + 4 * (8 * h + i);
                    sq[8 * h + i] += x[i].x * x[i].x + x[i].y * x[i].y + x[i].z * x[i].z + x[i].w * x[i].w;
                    *reinterpret_cast<uint2*>(box + r * 128 + ((((pl & 15) >> 1) ^ (r & 7)) << 4) + (pl & 1) * 8) =
                        make_uint2(lb_pack(x[i].x * w.x, x[i].y * w.y), lb_pack(x[i].z * w.z, x[i].w * w.w));
                }
            };
            float4 xa[8], xb[8];
            if (n_chunks > 0) load8(0, 0, xa);
            for (int c = 0; c < n_chunks; ++c) {
                const float4 w = load_w(c);
                load8(c, 1, xb);
                if (c >= ahead) {
                    if (!lb_bar_wait(empty0 + 8u * (c % stages), (unsigned)((c / stages) - 1) & 1u)) { ok = false; break; }
                    if (pt == 0) issue_w(c);
                }
                emit8(c, 0, xa, w, ssq);
                if (c + 1 < n_chunks) load8(c + 1, 0, xa);
                emit8(c, 1, xb, w, ssq);
                lb_bar_arrive(full0 + 8u * (c % stages));         // (release: the stores above are visible to who waits)
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float v = warp_sum(ssq[i]);
                if (pl == 0) ssq_tok[pw + 4 * i] = v;
            }
        }
        if (!ok) { atomicExch(status, 7); failed = 1; }
    } else {
        // ---------------------------------------------------------------- consumers
        const int rg = warp & 3, th = warp >> 2;
        const bool busy = 32 * th < M;                            // the second half of the tokens may be empty
        // ldmatrix: lanes 0-15 give the rows of the 16 x 16 piece of W at columns 0-7, lanes 16-31 at columns 8-15; for the
        // tokens, lanes 0-7 and 8-15 the two column halves of tokens 0-7, lanes 16-31 those of tokens 8-15
        const int a_row = lb_smem_row<EPI>(p, rg, lane & 15), b_row = 32 * th + (lane & 7) + ((lane >> 4) << 3);
        const unsigned a_off = (unsigned)(a_row * 128), a_x = (unsigned)(a_row & 7), a_u = (unsigned)(lane >> 4);
        const unsigned b_off = (unsigned)(2 * LB_BOX + b_row * 128), b_x = (unsigned)(b_row & 7), b_u = (unsigned)((lane >> 3) & 1);
        pdl_wait();
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c % stages;
            if (ok && !lb_bar_wait(full0 + 8u * s, (unsigned)(c / stages) & 1u)) { ok = false; if (lane == 0) { atomicExch(status, 7); failed = 1; } }
            if (ok && busy) {
                const unsigned base = mem0 + s * LB_STAGE;
                const int steps = (min(LB_KC, p.K - (c_begin + c) * LB_KC) + 15) / 16;     // (what a last step has beyond K is zeros)
#pragma unroll
                for (int kk = 0; kk < LB_KC / 16; ++kk) {
                    if (kk < steps) {
                        const unsigned box = (unsigned)(kk >> 2) * LB_BOX, u = (unsigned)(kk & 3) * 2;
                        unsigned a0, a1, a2, a3, b[8];
                        lb_ldmatrix4(base + box + a_off + (((u + a_u) ^ a_x) << 4), a0, a1, a2, a3);
                        lb_ldmatrix4(base + box + b_off + (((u + b_u) ^ b_x) << 4), b[0], b[1], b[2], b[3]);               // tokens 0-7 and 8-15 of the half
                        lb_ldmatrix4(base + box + b_off + 16 * 128 + (((u + b_u) ^ b_x) << 4), b[4], b[5], b[6], b[7]);    // tokens 16-23 and 24-31
#pragma unroll
                        for (int j = 0; j < 4; ++j) lb_mma(acc[j], a0, a1, a2, a3, b[2 * j], b[2 * j + 1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) lb_bar_arrive(empty0 + 8u * s);
        }
    }
    __syncthreads();                                             // the sums of squares are written; `failed` is final for this CTA
    ok = !failed;

    // acc[j][e] of lane (g, t) of consumer warp (rg, th): row g of the warp's low (e < 2) or high (e >= 2) group,
    // token 32 th + 8 j + 2 t + (e & 1)
    const int rg = warp & 3, th = warp >> 2;
    const bool writes = warp < LB_CONSUMERS && 32 * th < M && ks == 0;

    // What the epilogue needs besides the sums is loaded now, before the ranges are exchanged: the loads of 8 tokens in
    // flight together instead of one dependent chain a token behind the stores.
    const int half = EPI == LB_ROPE ? p.hd >> 1 : 1, pi = tile * 32 + rg * 8 + g;
    const int head = EPI == LB_ROPE ? pi / half : 0, d = pi - head * half;
    const bool row_in = EPI == LB_ROPE ? head < p.n_q + 2 * p.n_kv : true;
    const int n_lo = EPI == LB_ROPE ? head * p.hd + d : tile * LB_TW + 16 * rg + g, n_hi = EPI == LB_ROPE ? n_lo + half : n_lo + 8;
    float b_lo = 0.f, b_hi = 0.f, cs[8], sn[8];
    int pos[8], page[8];
    if (writes && EPI != LB_SWIGLU && p.bias && row_in) {
        if (n_lo < p.N) b_lo = load_as_f(p.bias, p.bias_dtype, n_lo);
        if (n_hi < p.N) b_hi = load_as_f(p.bias, p.bias_dtype, n_hi);
    }
    if (EPI == LB_ROPE) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int m = 32 * th + 8 * (i >> 1) + 2 * t + (i & 1);
            pos[i] = 0; page[i] = -1; cs[i] = 1.f; sn[i] = 0.f;
            if (writes && row_in && m < M) {
                pos[i] = p.tok_pos[m];
                if (head >= p.n_q && p.store) page[i] = p.block_table[(size_t)p.tok_row[m] * p.table_stride + pos[i] / PE_PAGE];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int m = 32 * th + 8 * (i >> 1) + 2 * t + (i & 1);
            if (writes && row_in && m < M && head < p.n_q + p.n_kv && p.cos_t) {
                cs[i] = p.cos_t[(size_t)pos[i] * half + d]; sn[i] = p.sin_t[(size_t)pos[i] * half + d];
            }
        }
    }

    if (SPLIT && ksplit > 1) {
        constexpr unsigned GATHER_BYTES = GATHER_FLOATS * 4;
        if (ks != 0) {
            // This range's sums go to the CTA of the first range: through this CTA's own shared memory (its stages are
            // free now) and from there in one bulk copy, which completes on that CTA's barrier.
            float* mine = reinterpret_cast<float*>(lb_mem);
            if (warp < LB_CONSUMERS) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) mine[((warp * 4 + j) * 4 + e) * 32 + lane] = ok ? acc[j][e] : 0.f;
            } else {
                const int pt = threadIdx.x - 32 * LB_CONSUMERS;
                if (pt < LB_TM) mine[LB_TW * LB_TM + pt] = (PRO == LB_RMSNORM && ok) ? ssq_tok[pt] : 0.f;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            lb_cluster_wait();                                   // every CTA of the cluster has set up its barrier
            if (threadIdx.x == 0) {
                unsigned dst, bar;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(lb_smem(gather + (size_t)(ks - 1) * GATHER_FLOATS)), "r"(0u));
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(gbar), "r"(0u));
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst), "r"(mem0), "r"(GATHER_BYTES), "r"(bar) : "memory");
            }
        } else {
            lb_cluster_wait();
            if (!lb_bar_wait(gbar, 0u)) { ok = false; if (threadIdx.x == 0) atomicExch(status, 7); }
            if (ok && warp < LB_CONSUMERS) {
                for (int o = 0; o < ksplit - 1; ++o) {           // in the order of the ranges
                    const float* src = gather + (size_t)o * GATHER_FLOATS;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[j][e] += src[((warp * 4 + j) * 4 + e) * 32 + lane];
                }
            }
        }
        // A CTA keeps its shared memory until the first CTA has received everything (the copies read it).
        lb_cluster_arrive();
        lb_cluster_wait();
    }
    if (!writes || !ok || !row_in) return;

    float rstd[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        rstd[i] = 1.f;
        if (PRO == LB_RMSNORM) {
            const int m = 32 * th + 8 * (i >> 1) + 2 * t + (i & 1);
            float s = ssq_tok[m];
            if (SPLIT && ksplit > 1)
                for (int o = 0; o < ksplit - 1; ++o) s += gather[(size_t)o * GATHER_FLOATS + LB_TW * LB_TM + m];
            rstd[i] = 1.0f / sqrtf(s / (float)p.K + p.eps);
        }
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int j = i >> 1, e = i & 1, m = 32 * th + 8 * j + 2 * t + e;
        if (m >= M) continue;
        float v_lo = acc[j][e] * rstd[i], v_hi = acc[j][2 + e] * rstd[i];
        if (EPI == LB_SWIGLU) {
            if (pi < p.I) {
                v_lo = lb_round(v_lo); v_hi = lb_round(v_hi);            // the unfused path rounds gate and up to bfloat16 first
                const float sig = 1.0f / (1.0f + expf(-v_lo));
                ((bf16*)p.out)[(size_t)m * p.I + pi] = __float2bfloat16_rn(v_lo * sig * v_hi);
            }
        } else if (EPI == LB_ROPE) {
            v_lo = lb_round(v_lo + b_lo); v_hi = lb_round(v_hi + b_hi);  // the unfused path rounds the projection before it rotates
            if (head < p.n_q + p.n_kv && p.cos_t) {
                const float a = v_lo * cs[i] - v_hi * sn[i], b = v_lo * sn[i] + v_hi * cs[i];
                v_lo = a; v_hi = b;
            }
            const bf16 o_lo = __float2bfloat16_rn(v_lo), o_hi = __float2bfloat16_rn(v_hi);
            if (head < p.n_q) {
                bf16* q = (bf16*)p.out + (size_t)m * p.n_q * p.hd + (size_t)head * p.hd;
                q[d] = o_lo; q[d + half] = o_hi;
            } else if (page[i] >= 0) {
                const bool is_k = head < p.n_q + p.n_kv;
                const int kvh = head - p.n_q - (is_k ? 0 : p.n_kv);
                bf16* dst = (is_k ? p.k_pool : p.v_pool) + (((size_t)page[i] * p.n_kv + kvh) * PE_PAGE + (pos[i] % PE_PAGE)) * p.hd;
                dst[d] = o_lo; dst[d + half] = o_hi;
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int n = h ? n_hi : n_lo;
                if (n >= p.N) continue;
                const float v = (h ? v_hi : v_lo) + (h ? b_hi : b_lo);
                if (EPI == LB_STORE) ((bf16*)p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
                else atomicAdd((float*)p.out + (size_t)m * p.N + n, v);  // the only sum into this element: a reduction in memory
            }
        }
    }
}

// ---------------------------------------------------------------- host side
extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }     // (this library's own copy of the switch)

static int lb_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

static size_t lb_gather_bytes(int ksplit) { return ksplit > 1 ? (size_t)(ksplit - 1) * (LB_TW * LB_TM + LB_TM) * 4 : 0; }
static int lb_stages(int ksplit, int chunks_per_split) {
    const size_t budget = 224 * 1024;
    int stages = (int)((budget - 1024 - lb_gather_bytes(ksplit)) / LB_STAGE);
    if (stages > LB_MAX_STAGES) stages = LB_MAX_STAGES;
    return stages > chunks_per_split ? chunks_per_split : stages;
}
static size_t lb_smem_bytes(int ksplit, int stages) { return (size_t)stages * LB_STAGE + lb_gather_bytes(ksplit) + 1024; }

template <int PRO, int EPI, bool SPLIT>
static int lb_allow_smem(size_t smem) {
    static size_t allowed = 0;
    if (smem > allowed) {
        PE_TRY(cudaFuncSetAttribute(linear_batch_kernel<PRO, EPI, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        allowed = smem;
    }
    return 0;
}

// How many clusters of `ksplit` CTAs the GPU runs at once (0: unknown).
template <int PRO, int EPI>
static int lb_clusters_at_once(int ksplit, int stages) {
    static int known[LB_MAX_SPLIT + 1][LB_MAX_STAGES + 1] = {};
    int& n = known[ksplit][stages];
    if (n) return n;
    const size_t smem = lb_smem_bytes(ksplit, stages);
    if (lb_allow_smem<PRO, EPI, true>(smem)) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ksplit * 64); cfg.blockDim = dim3(LB_THREADS); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int got = 0;
    if (cudaOccupancyMaxActiveClusters(&got, linear_batch_kernel<PRO, EPI, true>, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n = got;
}

template <int PRO, int EPI>
static int lb_launch(LbArgs& a, const void* A, const void* W, int box_rows, int tiles, int* status, cudaStream_t s) {
    if (!status) return PE_ERR_UNSUPPORTED;
    // Few tiles: cut K into ranges (chunks of 128 columns), one CTA each, up to 8 to a cluster, so that more SMs stream the
    // weights; but no more ranges than lets all clusters run at once (a GPU runs fewer CTAs in clusters than alone).
    const int chunks = (a.K + LB_KC - 1) / LB_KC;
    int split = 1;
    if (tiles * 2 <= lb_sm_count()) {
        split = lb_sm_count() / tiles;
        if (split > LB_MAX_SPLIT) split = LB_MAX_SPLIT;
        if (split > chunks) split = chunks;
        for (; split > 1; --split) {
            const int cps = (chunks + split - 1) / split, ks = (chunks + cps - 1) / cps;
            if (ks != split) continue;                            // (the same cut as fewer ranges)
            const int at_once = lb_clusters_at_once<PRO, EPI>(ks, lb_stages(ks, cps));
            if (at_once == 0 || at_once >= tiles) break;
        }
    }
    a.chunks_per_split = (chunks + split - 1) / split;
    a.ksplit = (chunks + a.chunks_per_split - 1) / a.chunks_per_split;
    a.stages = lb_stages(a.ksplit, a.chunks_per_split);
    if (a.stages < 1) return PE_ERR_UNSUPPORTED;
    CUtensorMap mw, ma;
    int rc = pe_tensor_map_2d(&mw, W, a.N, a.K, box_rows, 64, false);
    if (rc) return rc;
    ma = mw;
    if (PRO == LB_PLAIN && (rc = pe_tensor_map_2d(&ma, A, a.M, a.K, LB_TM, 64, false))) return rc;
    const size_t smem = lb_smem_bytes(a.ksplit, a.stages);
    if (a.ksplit > 1) {
        if (int e = lb_allow_smem<PRO, EPI, true>(smem)) return e;
        PE_TRY(pe_launch_cluster(linear_batch_kernel<PRO, EPI, true>, tiles * a.ksplit, LB_THREADS, smem, s, (unsigned)a.ksplit, mw, ma, a, status));
    } else {
        if (int e = lb_allow_smem<PRO, EPI, false>(smem)) return e;
        PE_TRY(pe_launch(linear_batch_kernel<PRO, EPI, false>, tiles, LB_THREADS, smem, s, mw, ma, a, status));
    }
    return 0;
}

static bool lb_aligned(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// x += a . W^T or out = a . W^T (+ bias); `a` bfloat16 [17 <= M <= 64, K], or with `x_norm` the float32 rows whose RMSNorm
// (weights norm_w, eps) is the operand.  epilogue: 1 store bfloat16, 2 add into float32 out.
extern "C" int pe_linear_batch(const void* a, const float* x_norm, const void* norm_w, int norm_w_dtype, float eps, const void* W,
                               const void* bias, int bias_dtype, void* out, int epilogue, int M, int N, int K, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > LB_TM || K <= 0 || K % 8 || (epilogue != 1 && epilogue != 2) || !lb_aligned(W) || !lb_aligned(x_norm ? (const void*)x_norm : a) ||
        (x_norm && !lb_aligned(norm_w)))
        return PE_ERR_UNSUPPORTED;
    LbArgs p = {};
    p.X = x_norm; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps;
    p.bias = bias; p.bias_dtype = bias_dtype; p.out = out; p.M = M; p.N = N; p.K = K;
    const int tiles = (N + LB_TW - 1) / LB_TW;
    cudaStream_t s = (cudaStream_t)stream;
    if (x_norm) return epilogue == 1 ? lb_launch<LB_RMSNORM, LB_STORE>(p, a, W, 64, tiles, status, s) : lb_launch<LB_RMSNORM, LB_ACCUM>(p, a, W, 64, tiles, status, s);
    return epilogue == 1 ? lb_launch<LB_PLAIN, LB_STORE>(p, a, W, 64, tiles, status, s) : lb_launch<LB_PLAIN, LB_ACCUM>(p, a, W, 64, tiles, status, s);
}

// act[M, I] = silu(h . Wg^T) * (h . Wu^T), h = RMSNorm(x); W = [Wg; Wu] is [2I, K].
extern "C" int pe_batch_norm_gate_up_swiglu(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* W, void* act,
                                            int M, int I, int K, int* status, void* stream) {
    if (M <= 0 || I <= 0) return 0;
    if (M > LB_TM || K <= 0 || K % 8 || !lb_aligned(W) || !lb_aligned(x) || !lb_aligned(norm_w)) return PE_ERR_UNSUPPORTED;
    LbArgs p = {};
    p.X = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps; p.out = act;
    p.M = M; p.N = 2 * I; p.K = K; p.I = I;
    return lb_launch<LB_RMSNORM, LB_SWIGLU>(p, nullptr, W, 32, (I + 31) / 32, status, (cudaStream_t)stream);
}

// q[M, n_q * hd] and the cache pages of keys and values from h = RMSNorm(x): project with W = [Wq; Wk; Wv], add bias, rotate
// q and k by position (cos_t null: no rotation), write keys and values at (page of the token's sequence, position).
extern "C" int pe_batch_norm_qkv_rope_store(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* W,
                                            const void* bias, int bias_dtype, void* q_out, int M, int K, int n_q, int n_kv, int hd,
                                            const float* cos_t, const float* sin_t, const int* tok_pos, const int* tok_row,
                                            void* k_pool, void* v_pool, const int* block_table, int table_stride, int store,
                                            int* status, void* stream) {
    if (M <= 0) return 0;
    if (M > LB_TM || K <= 0 || K % 8 || hd <= 0 || hd % 16 || !lb_aligned(W) || !lb_aligned(x) || !lb_aligned(norm_w) || !tok_pos ||
        (store && (!tok_row || !k_pool || !v_pool || !block_table)))
        return PE_ERR_UNSUPPORTED;
    LbArgs p = {};
    p.X = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps; p.bias = bias; p.bias_dtype = bias_dtype;
    p.out = q_out; p.M = M; p.N = (n_q + 2 * n_kv) * hd; p.K = K; p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.cos_t = cos_t; p.sin_t = sin_t;
    p.tok_pos = tok_pos; p.tok_row = tok_row; p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.block_table = block_table;
    p.table_stride = table_stride; p.store = store;
    const int half = hd / 2;
    p.run = half % 32 == 0 ? 32 : half % 16 == 0 ? 16 : 8;          // rows that lie together in W and in a tile's 32 pairs
    const int pairs = (n_q + 2 * n_kv) * half;
    return lb_launch<LB_RMSNORM, LB_ROPE>(p, nullptr, W, p.run, (pairs + 31) / 32, status, (cudaStream_t)stream);
}
