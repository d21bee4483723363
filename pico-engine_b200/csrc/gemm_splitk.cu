// out = A . W^T for 17 to 64 rows of A (a decode step of that many sequences) on the tcgen05 tensor cores, with K cut
// into ranges over a thread-block cluster: the products of a layer have 7 to 76 tiles of 128 rows of W, and one CTA a
// tile could not pull the weights through its SM fast enough (an SM takes about 64 bytes a cycle: 8.7 MB through 7 SMs
// are 30 us).  With the rows of W on the accumulator's 128 lanes and the tokens on its columns (M = 128, N = 64), the
// CTAs of a tile's ranges each stream their part of K, then hand one another the parts of the tile they do not finish
// themselves (a reduce-scatter through distributed shared memory: bulk copies shared -> shared::cluster, completing on
// the receiver's mbarrier), add what they received in the order of the ranges and run the epilogue on their own rows.
//
//   warp 0     one thread issues TMA tiled loads (128-byte swizzle) into a ring of stages: a box of W [128 rows x 64
//              columns] (before griddepcontrol.wait: no kernel writes weights) and a box of A [64 tokens x 64 columns]
//   warp 1     allocates tensor memory (four accumulators of 64 columns); one thread issues tcgen05.mma (four K = 16 steps a
//              stage, one to each accumulator: a chain of dependent 64-column MMAs ran at 300 cycles a step),
//              commits each stage's MMAs to the barrier that frees it, and the last to the accumulator's barrier
//   warps 2-5  read the accumulators (tcgen05.ld, 32 lanes a warp), store their sum as float32 [128 rows][64 tokens] in
//              shared memory (16-byte units XORed with the row so that neither the stores nor the later reads collide)
//              and exchange; then all six warps sum and finish this CTA's rows
//
// The 128 rows of a tile are two halves of 64: a CTA finishes rows [o h, (o + 1) h) of both (h = 64 / ranges), so that
// the rows that belong together lie with one CTA: plain rows n and n + 64 (STORE, ACCUM); gate row i and up row I + i
// (SWIGLU); dimension d of a head and d + hd / 2 (ROPE; the halves are then runs of 8 to 64 rows of W that lie
// together, fetched as boxes of their own).
//
//   epilogue  STORE     out[M, N] = acc (+ bias), bfloat16
//             ACCUM     x[M, N] += acc (+ bias) in float32 (the residual sum), a reduction in memory
//             SWIGLU    out[M, I] = silu(gate) * up
//             ROPE      bias, rotation of query and key heads by position, queries to out, keys and values to the cache
//
// Every wait on an mbarrier is bounded and gives up when another role has; a CTA that gave up still sends (zeros),
// arrives at its cluster barriers and frees its tensor memory, so that nothing is left waiting: *status becomes 8.
#include "common.cuh"
#include "tensor_map.cuh"

#define GS_BK 64
#define GS_BN 64                              // tokens: the accumulator's columns
#define GS_STAGE (128 * GS_BK * 2 + GS_BN * GS_BK * 2)
#define GS_MAX_STAGES 6
#define GS_THREADS 192
#define GS_TILE_BYTES (128 * GS_BN * 4)       // a tile of sums in shared memory
#define GS_MAX_SPLIT 8
#define GS_ACCS 4                               // accumulators in tensor memory: the K = 16 steps of a stage go to one each, so that
#define GS_TMEM_COLS (GS_ACCS * GS_BN)          // an MMA does not wait for the one before it (a chain of 64-column MMAs ran at 300 cycles a step)
#define GS_WAIT_CYCLES 2000000000ll

enum { GS_STORE = 0, GS_ACCUM = 1, GS_SWIGLU = 2, GS_ROPE = 3 };

struct GsArgs {
    void* out; const void* bias; int bias_dtype;
    int M, N, K;
    int ksplit, blocks_per_split, stages;
    int I;
    int n_q, n_kv, hd, run;
    const float* cos_t; const float* sin_t;
    const int* tok_pos; const int* tok_row;
    bf16* k_pool; bf16* v_pool; const int* block_table; int table_stride; int store;
};

__device__ __forceinline__ unsigned gs_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool gs_wait(unsigned bar, unsigned parity, const volatile int* abort_flag) {
    unsigned done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    const long long deadline = clock64() + GS_WAIT_CYCLES;
    for (unsigned spins = 1;; ++spins) {
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((spins & 63u) == 0 && (*abort_flag || clock64() > deadline)) return false;
    }
}
// K-major operand tile [rows][64 bfloat16] in 128-byte swizzle: 8-row groups are 1024 bytes apart
__device__ __forceinline__ unsigned long long gs_desc(unsigned smem_addr) {
    return (unsigned long long)((smem_addr >> 4) & 0x3FFFu) | ((unsigned long long)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void gs_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void gs_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gs_ld32(unsigned taddr, float (&v)[32]) {
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
__device__ __forceinline__ float gs_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void gs_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void gs_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ void gs_epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }    // the four epilogue warps

// Element (row, m) of a tile of sums: 16-byte units XORed with the row.
__device__ __forceinline__ int gs_at(int row, int m) { return row * GS_BN + ((((m >> 2) ^ (row & 15)) << 2) | (m & 3)); }

// The rows of W that row j (0..63) of half `hf` of tile `tile` stands for: the output feature, or -1.
template <int EPI>
__device__ __forceinline__ int gs_feature(const GsArgs& p, int tile, int hf, int j) {
    if (EPI == GS_SWIGLU) { const int i = tile * 64 + j; return i < p.I ? (hf ? p.I + i : i) : -1; }
    if (EPI == GS_ROPE) {
        const int half = p.hd >> 1, pi = tile * 64 + j, head = pi / half;
        return head < p.n_q + 2 * p.n_kv ? head * p.hd + (pi - head * half) + (hf ? half : 0) : -1;
    }
    const int n = tile * 128 + hf * 64 + j;
    return n < p.N ? n : -1;
}

template <int EPI>
__global__ void __launch_bounds__(GS_THREADS, 1) gemm_splitk_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ CUtensorMap map_a, const GsArgs p, int* status) {
    extern __shared__ unsigned char gs_raw[];
    __shared__ __align__(8) unsigned long long full_bar[GS_MAX_STAGES], empty_bar[GS_MAX_STAGES], acc_bar, gather_bar;
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.ksplit, rank = blockIdx.x, tile = blockIdx.y, stages = p.stages;        // the cluster is the grid's x
    const int k_blocks_all = (p.K + GS_BK - 1) / GS_BK;
    const int kb0 = rank * p.blocks_per_split, kb1 = min(k_blocks_all, kb0 + p.blocks_per_split), n_kb = max(0, kb1 - kb0);
    const unsigned stage0 = (gs_smem(gs_raw) + 1023u) & ~1023u;
    unsigned char* const mem = gs_raw + (stage0 - gs_smem(gs_raw));
    float* const mine = reinterpret_cast<float*>(mem + (size_t)stages * GS_STAGE);           // this CTA's sums of the whole tile
    float* const recv = mine + 128 * GS_BN;                                                   // [sender slot][half][h rows][64]
    const int h = 64 / S;                                                                     // rows of a half that a CTA finishes
    const volatile int* abort_flag = &abort_s;
    const unsigned gbar = gs_smem(&gather_bar);

    if (threadIdx.x == 32) {                                 // the copies' descriptors, fetched while the barriers are set up
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    }
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gs_smem(&full_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gs_smem(&empty_bar[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gs_smem(&acc_bar)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gbar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (S > 1) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gbar), "r"((unsigned)((S - 1) * 2 * h * GS_BN * 4)) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gs_smem(&tmem_base_s)), "r"((unsigned)GS_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_base_s;
    if (S > 1) gs_cluster_arrive();                          // waited for before the first copy into another CTA
    pdl_launch_dependents();                                 // (only now: a successor that took tensor memory first could starve this allocation)

    if (warp == 0) {
        if (lane == 0) {                                     // ---------------- producer
            // the boxes of W of a stage: the tile's two halves, each in runs of rows that lie together in W
            const int run = EPI == GS_ROPE ? p.run : 64;
            auto load_w = [&](int i) {
                const int s = i % stages;
                const unsigned dst = stage0 + s * GS_STAGE, bar = gs_smem(&full_bar[s]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((unsigned)GS_STAGE) : "memory");
                for (int hf = 0; hf < 2; ++hf)
                    for (int j = 0; j < 64; j += run) {
                        int y;
                        if (EPI == GS_SWIGLU) y = tile * 64 + j + (hf ? p.I : 0);
                        else if (EPI == GS_ROPE) {
                            const int half = p.hd >> 1, pi = tile * 64 + j, head = pi / half;
                            y = head * p.hd + (pi - head * half) + (hf ? half : 0);          // (past the last head: past N, read as zeros)
                        } else y = tile * 128 + hf * 64 + j;
                        pe_tma_load_2d(dst + (hf * 64 + j) * 128, &map_w, (kb0 + i) * GS_BK, y, bar);
                    }
            };
            auto load_a = [&](int i) {
                const int s = i % stages;
                pe_tma_load_2d(stage0 + s * GS_STAGE + 128 * GS_BK * 2, &map_a, (kb0 + i) * GS_BK, 0, gs_smem(&full_bar[s]));
            };
            const int ahead = min(n_kb, stages);
            for (int i = 0; i < ahead; ++i) load_w(i);       // weights: nothing to wait for
            pdl_wait();
            for (int i = 0; i < ahead; ++i) load_a(i);
            for (int i = ahead; i < n_kb; ++i) {
                if (!gs_wait(gs_smem(&empty_bar[i % stages]), (unsigned)((i / stages) - 1) & 1u, abort_flag)) { atomicExch(status, 8); abort_s = 1; break; }
                load_w(i);
                load_a(i);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                     // ---------------- MMA issuer
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = 64, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(GS_BN >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % stages;
                if (!gs_wait(gs_smem(&full_bar[s]), (unsigned)(i / stages) & 1u, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned base = stage0 + s * GS_STAGE;
                const unsigned long long da = gs_desc(base), db = gs_desc(base + 128 * GS_BK * 2);
#pragma unroll
                for (int kk = 0; kk < GS_BK / 16; ++kk)       // 16 columns = 32 bytes further inside the swizzle atom
                    gs_mma(tmem + (unsigned)((kk % GS_ACCS) * GS_BN), da + 2ull * kk, db + 2ull * kk, idesc, i > 0 ? 1u : 0u);
                gs_commit(gs_smem(&empty_bar[s]));            // the stage is free once these MMAs have read it
            }
            if (ok) gs_commit(gs_smem(&acc_bar));
            else { atomicExch(status, 8); abort_s = 1; }
        }
    } else {                                                 // ---------------- epilogue, warps 2..5
        const int quarter = warp & 3;
        pdl_wait();
        bool ok = n_kb == 0 || gs_wait(gs_smem(&acc_bar), 0u, abort_flag);
        if (!ok) { atomicExch(status, 8); abort_s = 1; }
        {   // this thread's row of the accumulator into the tile of sums (zeros if the range is empty or the wait gave up)
            const int row = quarter * 32 + lane;
            float v[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                if (ok && n_kb > 0) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    gs_ld32(tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)(c * 32), v);
#pragma unroll
                    for (int a = 1; a < GS_ACCS; ++a) {       // the accumulators, added in their order
                        float w[32];
                        gs_ld32(tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)(a * GS_BN + c * 32), w);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] += w[i];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    *reinterpret_cast<float4*>(mine + gs_at(row, c * 32 + u * 4)) = make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
            }
        }
        if (S > 1) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            gs_epilogue_sync();
            gs_cluster_wait();                               // every CTA of the cluster has set up its barrier
            if (lane == 0) {
                // rows [q h, (q + 1) h) of both halves go to CTA q; a sender's slot there: its rank, counted without q
                // (a thread issues its copies one after the other: the four warps share them)
                for (int q = warp - 2; q < S; q += 4) {
                    if (q == rank) continue;
                    const int slot = rank < q ? rank : rank - 1;
                    for (int hf = 0; hf < 2; ++hf) {
                        unsigned dst, bar;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(gs_smem(recv + ((size_t)(slot * 2 + hf) * h) * GS_BN)), "r"((unsigned)q));
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(gbar), "r"((unsigned)q));
                        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst), "r"(gs_smem(mine + (size_t)(hf * 64 + q * h) * GS_BN)), "r"((unsigned)(h * GS_BN * 4)), "r"(bar) : "memory");
                    }
                }
            }
            if (!gs_wait(gbar, 0u, abort_flag)) { ok = false; atomicExch(status, 8); abort_s = 1; }
        }
    }
    if (S > 1 && warp < 2) gs_cluster_wait();                // (the epilogue warps have waited already)
    __syncthreads();                                         // the tile of sums is complete, and what the other ranges sent is here
    {
        bool ok = !abort_s;
        const int etid = threadIdx.x;

        // ---- this CTA's rows: j in [rank h, (rank + 1) h) of both halves, all tokens; sums in the order of the ranges.
        // A thread takes four tokens (a 16-byte unit) of a row at a time.
        auto total4 = [&](int hf, int j, int u) {            // j: row within the half; u: unit = tokens 4 u .. 4 u + 3
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int off = ((u ^ (j & 15)) << 2);
#pragma unroll
            for (int r = 0; r < GS_MAX_SPLIT; ++r) {
                if (r < S) {
                    const float* src = r == rank ? mine + (hf * 64 + j) * GS_BN
                                                 : recv + ((size_t)(((r < rank ? r : r - 1) * 2 + hf) * h) + (j - rank * h)) * GS_BN;
                    const float4 t4 = *reinterpret_cast<const float4*>(src + off);
                    v.x += t4.x; v.y += t4.y; v.z += t4.z; v.w += t4.w;
                }
            }
            return v;
        };
        if (ok) {
            if (EPI == GS_STORE || EPI == GS_ACCUM) {
                // consecutive threads: consecutive rows (features) of the two halves, then the next unit of tokens
                for (int idx = etid; idx < 2 * h * (GS_BN / 4); idx += GS_THREADS) {
                    const int jj = idx % h, hf = (idx / h) & 1, u = idx / (2 * h), j = rank * h + jj;
                    const int n = gs_feature<EPI>(p, tile, hf, j);
                    if (4 * u >= p.M || n < 0) continue;
                    const float4 v4 = total4(hf, j, u);
                    const float b = p.bias ? load_as_f(p.bias, p.bias_dtype, n) : 0.f;
                    const float v[4] = {v4.x + b, v4.y + b, v4.z + b, v4.w + b};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int m = 4 * u + i;
                        if (m >= p.M) break;
                        if (EPI == GS_STORE) ((bf16*)p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v[i]);
                        else atomicAdd((float*)p.out + (size_t)m * p.N + n, v[i]);   // the only sum into this element: a reduction in memory
                    }
                }
            } else {
                for (int idx = etid; idx < h * (GS_BN / 4); idx += GS_THREADS) {
                    const int jj = idx % h, u = idx / h, j = rank * h + jj;
                    const int n_lo = gs_feature<EPI>(p, tile, 0, j), n_hi = gs_feature<EPI>(p, tile, 1, j);
                    if (4 * u >= p.M || n_lo < 0) continue;
                    const float4 lo4 = total4(0, j, u), hi4 = total4(1, j, u);
                    const float lo[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hi[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
                    if (EPI == GS_SWIGLU) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int m = 4 * u + i;
                            if (m >= p.M) break;
                            const float g = gs_round(lo[i]), up = gs_round(hi[i]);       // the unfused path rounds gate and up to bfloat16 first
                            float e, rcp;
                            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
                            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(1.0f + e));
                            ((bf16*)p.out)[(size_t)m * p.I + n_lo] = __float2bfloat16_rn(g * rcp * up);
                        }
                    } else {
                        const int half = p.hd >> 1, head = n_lo / p.hd, d = n_lo - head * p.hd;
                        const float b_lo = p.bias ? load_as_f(p.bias, p.bias_dtype, n_lo) : 0.f, b_hi = p.bias ? load_as_f(p.bias, p.bias_dtype, n_hi) : 0.f;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int m = 4 * u + i;
                            if (m >= p.M) break;
                            float v_lo = gs_round(lo[i] + b_lo), v_hi = gs_round(hi[i] + b_hi);   // the unfused path rounds the projection before it rotates
                            const int pos = p.tok_pos[m];
                            if (head < p.n_q + p.n_kv && p.cos_t) {
                                const float cs = p.cos_t[(size_t)pos * half + d], sn = p.sin_t[(size_t)pos * half + d];
                                const float a = v_lo * cs - v_hi * sn, b = v_lo * sn + v_hi * cs;
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
                                    bf16* dst = (is_k ? p.k_pool : p.v_pool) + (((size_t)page * p.n_kv + kvh) * PE_PAGE + (pos % PE_PAGE)) * p.hd;
                                    dst[d] = o_lo; dst[d + half] = o_hi;
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    if (S > 1) {
        gs_cluster_arrive();                                 // a CTA keeps its shared memory until every CTA has what it sent
        gs_cluster_wait();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)GS_TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
static int gs_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

static size_t gs_smem_bytes(int ksplit, int stages) {
    return 1024 + (size_t)stages * GS_STAGE + GS_TILE_BYTES + (ksplit > 1 ? (size_t)(ksplit - 1) * 2 * (64 / ksplit) * GS_BN * 4 : 0);
}
static int gs_stages(int ksplit, int blocks) {
    int stages = (int)((224 * 1024 - gs_smem_bytes(ksplit, 0)) / GS_STAGE);
    if (stages > GS_MAX_STAGES) stages = GS_MAX_STAGES;
    return stages > blocks ? blocks : stages;
}

template <int EPI>
static int gs_allow_smem(size_t smem) {
    static size_t allowed = 0;
    if (smem > allowed) {
        PE_TRY(cudaFuncSetAttribute(gemm_splitk_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        allowed = smem;
    }
    return 0;
}

// How many clusters of `ksplit` CTAs the GPU runs at once (0: unknown).
template <int EPI>
static int gs_clusters_at_once(int ksplit, int stages) {
    static int known[GS_MAX_SPLIT + 1][GS_MAX_STAGES + 1] = {};
    int& n = known[ksplit][stages];
    if (n) return n;
    const size_t smem = gs_smem_bytes(ksplit, stages);
    if (gs_allow_smem<EPI>(smem)) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ksplit, 64); cfg.blockDim = dim3(GS_THREADS); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int got = 0;
    if (cudaOccupancyMaxActiveClusters(&got, gemm_splitk_kernel<EPI>, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n = got;
}

template <int EPI>
static int gs_launch(GsArgs& a, const void* A, const void* W, int box_rows, int tiles, int* status, cudaStream_t s) {
    if (!status) return PE_ERR_UNSUPPORTED;
    // As many ranges of K (1, 2, 4 or 8: what divides the 64 rows of a half) as keeps all clusters running at once.
    const int blocks = (a.K + GS_BK - 1) / GS_BK;
    int split = GS_MAX_SPLIT;
    for (; split > 1; split >>= 1) {
        if (split > blocks || tiles * split > gs_sm_count()) continue;
        const int per = (blocks + split - 1) / split;
        if ((blocks + per - 1) / per != split) continue;     // (a range would be empty)
        const int at_once = gs_clusters_at_once<EPI>(split, gs_stages(split, per));
        if (at_once == 0 || at_once >= tiles) break;
    }
    a.ksplit = split;
    a.blocks_per_split = (blocks + split - 1) / split;
    a.stages = gs_stages(split, a.blocks_per_split);
    if (a.stages < 1) return PE_ERR_UNSUPPORTED;
    CUtensorMap mw, ma;
    int rc = pe_tensor_map_2d(&mw, W, a.N, a.K, box_rows, GS_BK, false);
    if (rc) return rc;
    if ((rc = pe_tensor_map_2d(&ma, A, a.M, a.K, GS_BN, GS_BK, false))) return rc;
    const size_t smem = gs_smem_bytes(split, a.stages);
    if (int e = gs_allow_smem<EPI>(smem)) return e;
    PE_TRY(pe_launch_cluster(gemm_splitk_kernel<EPI>, dim3(split, tiles), GS_THREADS, smem, s, (unsigned)split, mw, ma, a, status));
    return 0;
}

static bool gs_aligned(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// epilogue 0: out bfloat16 [M, N] = A . W^T + bias;  1: float32 out [M, N] += A . W^T (+ bias);
//          2: out bfloat16 [M, N / 2] = silu(A . Wg^T) * (A . Wu^T), W = [Wg; Wu];  M <= 64
extern "C" int pe_gemm_splitk(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                              int M, int N, int K, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > GS_BN || K <= 0 || K % 8 || epilogue < 0 || epilogue > 2 || !gs_aligned(A) || !gs_aligned(W) || (epilogue == 2 && (N % 2 || bias)))
        return PE_ERR_UNSUPPORTED;
    GsArgs p = {};
    p.out = out; p.bias = bias; p.bias_dtype = bias_dtype; p.M = M; p.N = N; p.K = K; p.I = N / 2;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == 0) return gs_launch<GS_STORE>(p, A, W, 64, (N + 127) / 128, status, s);
    if (epilogue == 1) return gs_launch<GS_ACCUM>(p, A, W, 64, (N + 127) / 128, status, s);
    return gs_launch<GS_SWIGLU>(p, A, W, 64, (p.I + 63) / 64, status, s);
}

// q[M, n_q * hd] and the cache pages of keys and values from A [M <= 64, K]: project with W = [Wq; Wk; Wv], add bias,
// rotate q and k by position (cos_t null: no rotation), write keys and values at (page of the token's sequence, position).
extern "C" int pe_gemm_splitk_rope(const void* A, const void* W, const void* bias, int bias_dtype, void* q_out, int M, int K,
                                   int n_q, int n_kv, int hd, const float* cos_t, const float* sin_t, const int* tok_pos,
                                   const int* tok_row, void* k_pool, void* v_pool, const int* block_table, int table_stride,
                                   int store, int* status, void* stream) {
    if (M <= 0) return 0;
    if (M > GS_BN || K <= 0 || K % 8 || hd <= 0 || hd % 16 || !gs_aligned(A) || !gs_aligned(W) || !tok_pos ||
        (store && (!tok_row || !k_pool || !v_pool || !block_table)))
        return PE_ERR_UNSUPPORTED;
    GsArgs p = {};
    p.out = q_out; p.bias = bias; p.bias_dtype = bias_dtype; p.M = M; p.N = (n_q + 2 * n_kv) * hd; p.K = K;
    p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.cos_t = cos_t; p.sin_t = sin_t; p.tok_pos = tok_pos; p.tok_row = tok_row;
    p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.block_table = block_table; p.table_stride = table_stride; p.store = store;
    const int half = hd / 2;
    p.run = half % 64 == 0 ? 64 : half % 32 == 0 ? 32 : half % 16 == 0 ? 16 : 8;     // rows that lie together in W and in a tile's 64 pairs
    const int pairs = (n_q + 2 * n_kv) * half;
    return gs_launch<GS_ROPE>(p, A, W, p.run, (pairs + 63) / 64, status, (cudaStream_t)stream);
}
