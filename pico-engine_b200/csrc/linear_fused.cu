// The matrix products of a decode step for up to 16 rows (sequences), each fused with what
// stands before and after it in the layer, so that a layer is five kernels instead of ten:
//
//   prologue  PLAIN     A is bfloat16 [M, K]
//             RMSNORM   A = RMSNorm(x) of the float32 residual stream x: bfloat16(x * w) is multiplied and
//                       rsqrt(mean(x^2) + eps) applied to the sums, so x is read once
//   epilogue  STORE     out[M, N] = acc (+ bias), bfloat16 or float32
//             ACCUM     x[M, N] += acc (+ bias) in float32 (the residual sum)
//             SWIGLU    out[M, I] = silu(gate) * up, gate and up being rows i and I + i of W
//             ROPE      rows are query, key and value heads: add bias, rotate query and key heads
//                       by position, write queries to out and keys and values into the paged cache
//
// At these sizes a product is bound by memory latency, not bandwidth: what counts is how many
// bytes are in flight and how few dependent trips to memory a kernel makes.  A CTA of eight
// warps owns 8 or 16 rows of W over all of K, or, where K is long and the rows are few (the
// down projection), over one of `ksplit` ranges of K: the CTAs of the ranges of a tile are a
// thread-block cluster, and the others send their sums into the first one's shared memory
// (st.async, counted on an mbarrier there), which adds them in the order of the ranges and
// runs the epilogue; there is no second pass over global memory.  Its
// rows are brought into shared memory by bulk asynchronous copies (cp.async.bulk, the 1-D TMA
// path, completing on an mbarrier), one copy per row and chunk of up to 1024 columns, up to
// four chunks in flight; registers hold none of it, so many CTAs are resident and the whole
// matrix can be under way at once.  The rows are dealt out to all eight warps, four to each: a warp issues
// its copies one after the other, at about 65 cycles a copy.  The copies are issued before the kernel waits for its
// predecessor (griddepcontrol.wait): no kernel writes weights.  The roles of the MMA operands
// are swapped as in linear_mma.cu: rows of W are the M side of mma.sync m16n8k16, sequences
// the N side; the warps take the 32-wide k steps of a chunk in turn and add their partial sums
// in shared memory in the order of the warps.  The 16 rows of a tile are two groups of 8: for
// SWIGLU the matching gate and up rows, for ROPE the two halves of a head that rotate
// together, so the epilogue finds its pairs in one CTA.
//
// Waiting on an mbarrier is bounded: a wait that runs out sets *status to 1 and the CTA
// returns, leaving its outputs unwritten; the host reads the status word with its results.
//
// pico-engine runs these as separate launches: rmsnorm, F.linear, rope, index_copy_, addmm,
// silu_mul (src/pico_engine/model.py:175-235).
#include "common.cuh"

#define LF_WARPS 8
#define LF_UNROLL(NT) ((NT) == 1 ? 4 : 2)   // k steps of a chunk a warp takes: what its registers hold of the activations
#define LF_MAX_CHUNK 1024            // columns of W per bulk copy (LF_WARPS * LF_UNROLL * 32 at most)
#define LF_MAX_STAGES 4              // chunks in flight: as many as fit in 160 KB of shared memory, at most twice this
#define LF_ROW_PAD 8                 // bfloat16 of padding per row in shared memory: skews the banks
#define LF_WAIT_CYCLES 2000000000ll    // about a second of SM clock: the longest a CTA waits for its own copies

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
    int chunk, stages;        // columns per bulk copy (a multiple of 32) and copies in flight per row
    int ksplit, kc;           // STORE/ACCUM: ranges of K a tile is cut into (CTAs of a cluster) and columns per range
    int I;                    // SWIGLU
    // ROPE
    int n_q, n_kv, hd;
    const float* cos_t; const float* sin_t;
    const int* tok_pos; const int* tok_row;
    bf16* k_pool; bf16* v_pool; const int* block_table; int table_stride; int store;
};

__device__ __forceinline__ unsigned lf_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lf_bar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void lf_bar_expect(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lf_bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// true when the phase with this parity has completed; false when the wait ran out
__device__ __forceinline__ bool lf_bar_wait(unsigned bar, unsigned parity) {
    const long long deadline = clock64() + LF_WAIT_CYCLES;
    for (;;) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() > deadline) return false;
        __nanosleep(40);
    }
}
__device__ __forceinline__ void lf_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void lf_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// a float into the shared memory of CTA `rank` of the cluster, at the address it has here; its 4 bytes
// are counted on that CTA's mbarrier
__device__ __forceinline__ void lf_send(unsigned local_addr, float v, unsigned local_bar, unsigned rank) {
    unsigned addr, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(local_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(addr), "r"(__float_as_uint(v)), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lf_lds16(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
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

// CTAs resident per SM that the register budget is set for: the products with many tiles (gate and up,
// the vocabulary) want as many as their shared memory allows; q/k/v has fewer tiles than the GPU has SMs
// and takes the registers instead.
#define LF_MIN_CTAS(NT, RT, EPI) ((RT) == 2 ? 3 : (EPI) == LF_ROPE ? ((NT) == 1 ? 3 : 2) : ((NT) == 1 ? 5 : 3))

// NT: 8-row tiles of sequences (M <= 8 * NT); RT: 16-row tiles of W a CTA takes (2 where a product has
// so many tiles that the activations, which every CTA reads, would cost as much as the weights);
// SPLIT: a tile's K is cut into ranges over a cluster
template <int NT, int RT, int PRO, int EPI, bool SPLIT>
__global__ void __launch_bounds__(32 * LF_WARPS, LF_MIN_CTAS(NT, RT, EPI)) linear_fused_kernel(const LfArgs p, int* status) {
    extern __shared__ __align__(128) unsigned char lf_smem[];   // [stage][16 * RT rows][chunk + pad] bfloat16
    __shared__ __align__(8) unsigned long long bars[2 * LF_MAX_STAGES], bars_a[2 * LF_MAX_STAGES], bar_x;
    __shared__ float ssq[LF_WARPS][NT * 8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int M = p.M;
    // the range of K of this CTA (all of it unless the tile is split over a cluster) and its tile
    const int ksplit = SPLIT ? p.ksplit : 1;
    const int tile = ksplit > 1 ? blockIdx.x / ksplit : blockIdx.x, ks = ksplit > 1 ? blockIdx.x % ksplit : 0;
    const int k_begin = ks * p.kc, K = min(p.K, k_begin + p.kc) - k_begin;      // K: columns of this CTA's range

    // the rows of W of this tile: group lo feeds MMA rows 0-7, group hi rows 8-15 (hi_base < 0: none);
    // with RT = 2 the second 16-row tile follows at lo_base + rt_step, hi_base + rt_step
    int lo_base, hi_base;
    const int rt_step = EPI == LF_SWIGLU ? 8 : 16;
    if (EPI == LF_SWIGLU) {
        lo_base = blockIdx.x * 8 * RT; hi_base = p.I + lo_base;
    } else if (EPI == LF_ROPE) {
        const int half = p.hd >> 1, per_head = half >> 3;
        lo_base = (blockIdx.x / per_head) * p.hd + (blockIdx.x % per_head) * 8; hi_base = lo_base + half;
    } else {
        lo_base = tile * p.rows * RT; hi_base = p.rows == 16 ? lo_base + 8 : -1;
    }
    const int chunk = p.chunk, n_chunks = (K + chunk - 1) / chunk, stages = p.stages;
    const int tile_rows = hi_base < 0 ? 8 : 16 * RT;         // rows of the tile held in shared memory
    const int a_rows = PRO == LF_PLAIN ? NT * 8 : 0;         // PLAIN: the activations of a chunk are staged beside W
    const unsigned row_bytes = (unsigned)(chunk + LF_ROW_PAD) * 2u, stage_bytes = (unsigned)(tile_rows + a_rows) * row_bytes;
    const unsigned smem0 = lf_smem_addr(lf_smem), bar0 = lf_smem_addr(bars), bar_a0 = lf_smem_addr(bars_a);
    const unsigned bar_x0 = lf_smem_addr(&bar_x);
    // what the other ranges send: [range - 1][item][low sum, high sum, sum of squares], behind the stages
    // The warps' partial sums.  For 9 to 16 rows (16 KB with two row tiles) they take the place of the stages once every
    // warp is done with them, so that three CTAs fit an SM; for up to 8 rows they have their own array and no warp waits.
    constexpr bool RED_IN_RING = NT > 1;
    __shared__ float red_own[RED_IN_RING ? 1 : LF_WARPS][RT * NT * 4][32];
    float (*red)[RT * NT * 4][32] = RED_IN_RING ? reinterpret_cast<float (*)[RT * NT * 4][32]>(lf_smem) : red_own;
    constexpr unsigned RED_BYTES = RED_IN_RING ? LF_WARPS * RT * NT * 4 * 32 * 4 : 0;
    float* gather = reinterpret_cast<float*>(lf_smem + max((unsigned)stages * stage_bytes, RED_BYTES));

    // row rr of the tile in shared memory (16 a tile: 8 of group lo, 8 of group hi) holds this row of W, or zeros
    const int my_rt = lane >> 4, my_l = lane & 15;
    const int my_row = my_l < 8 ? lo_base + my_rt * rt_step + my_l : (hi_base < 0 ? -1 : hi_base + my_rt * rt_step + my_l - 8);
    const bool my_row_ok = lane < tile_rows && my_row >= 0 && my_row < p.N &&
                           (EPI != LF_SWIGLU || my_l >= 8 || my_row < p.I);   // a gate row past I is no gate row

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { lf_bar_init(bar0 + 8u * s, 1u); lf_bar_init(bar_a0 + 8u * s, 1u); }
        lf_bar_init(bar_x0, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (ksplit > 1 && ks == 0) lf_bar_expect(bar_x0, (unsigned)((ksplit - 1) * M * 8 * 3 * 4));
    }
    if (warp == 1 && lane < tile_rows && !my_row_ok) {     // rows that no copy fills read as zeros
        for (int s = 0; s < stages; ++s)
            for (unsigned o = 0; o < row_bytes; o += 16)
                *reinterpret_cast<uint4*>(lf_smem + s * stage_bytes + lane * row_bytes + o) = make_uint4(0u, 0u, 0u, 0u);
    }
    const bool my_a_ok = lane < a_rows && lane < M;          // row m of A is copied (else it reads as zeros)
    if (warp == 2 && lane < a_rows && !my_a_ok) {
        for (int s = 0; s < stages; ++s)
            for (unsigned o = 0; o < row_bytes; o += 16)
                *reinterpret_cast<uint4*>(lf_smem + s * stage_bytes + (tile_rows + lane) * row_bytes + o) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    if (ksplit > 1) lf_cluster_arrive();                     // waited for before the first write to another CTA

    // Chunk c of every valid row into stage c % stages; called by all threads.  A thread's bulk copies are issued one
    // after the other at about 65 cycles each (measured), the lanes of a warp instruction too, so the rows are dealt out
    // to the warps: lanes 0-3 of warp w copy rows 4 w .. 4 w + 3 of W, lanes 4-5 rows 2 w, 2 w + 1 of the activations.
    const int cp_r = lane < 4 ? warp * 4 + lane : -1;
    const int cp_rt = cp_r >> 4, cp_l = cp_r & 15;
    const int cp_row = cp_r < 0 ? -1 : cp_l < 8 ? lo_base + cp_rt * rt_step + cp_l : (hi_base < 0 ? -1 : hi_base + cp_rt * rt_step + cp_l - 8);
    const bool cp_ok = cp_r >= 0 && cp_r < tile_rows && cp_row >= 0 && cp_row < p.N && (EPI != LF_SWIGLU || cp_l >= 8 || cp_row < p.I);
    const unsigned n_ok = __popc(__ballot_sync(0xffffffffu, my_row_ok));
    auto issue = [&](int c) {
        const int k0 = c * chunk, cols = min(chunk, K - k0);
        const unsigned bar = bar0 + 8u * (c % stages);
        if (threadIdx.x == 0) lf_bar_expect(bar, n_ok * (unsigned)cols * 2u);
        if (cp_ok) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier reads of the stage precede its refill
            lf_bulk_copy(smem0 + (c % stages) * stage_bytes + cp_r * row_bytes, p.W + (size_t)cp_row * p.K + k_begin + k0,
                         (unsigned)cols * 2u, bar);
        }
    };

    // the same for the activations (PLAIN only), after the wait for the predecessor
    const int cp_a = (lane == 4 || lane == 5) ? warp * 2 + lane - 4 : -1;
    const bool cp_a_ok = cp_a >= 0 && cp_a < a_rows && cp_a < M;
    const unsigned n_a_ok = __popc(__ballot_sync(0xffffffffu, my_a_ok));
    auto issue_a = [&](int c) {
        const int k0 = c * chunk, cols = min(chunk, K - k0);
        const unsigned bar = bar_a0 + 8u * (c % stages);
        if (threadIdx.x == 0) lf_bar_expect(bar, n_a_ok * (unsigned)cols * 2u);
        if (cp_a_ok) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            lf_bulk_copy(smem0 + (c % stages) * stage_bytes + (tile_rows + cp_a) * row_bytes, p.A + (size_t)cp_a * p.K + k_begin + k0,
                         (unsigned)cols * 2u, bar);
        }
    };

    pdl_launch_dependents();
    for (int c = 0; c < n_chunks && c < stages; ++c) issue(c);      // W first: no kernel writes it, so it need not wait
    // ROPE: what the epilogue needs of the step's description (positions, pages) and of the rotation tables is
    // asked for now: none of it is written by a kernel of the step, and the epilogue then waits for no load.
    int ep_pos = 0, ep_page = -1;
    float ep_cos = 1.f, ep_sin = 0.f;
    if (EPI == LF_ROPE && threadIdx.x < NT * 64) {
        const int idx = threadIdx.x, j = idx >> 6, e1 = (idx >> 5) & 1, ln = idx & 31;
        const int r = ln >> 2, m = j * 8 + 2 * (ln & 3) + e1;
        if (m < M) {
            const int half = p.hd >> 1, per_head = half >> 3;
            const int head = blockIdx.x / per_head, d = (blockIdx.x % per_head) * 8 + r;
            ep_pos = p.tok_pos[m];
            if (head < p.n_q + p.n_kv && p.cos_t) { ep_cos = p.cos_t[(size_t)ep_pos * half + d]; ep_sin = p.sin_t[(size_t)ep_pos * half + d]; }
            if (head >= p.n_q && p.store) ep_page = p.block_table[(size_t)p.tok_row[m] * p.table_stride + ep_pos / PE_PAGE];
        }
    }
    pdl_wait();                                              // from here on the preceding kernel's results may be read
    if (PRO == LF_PLAIN)
        for (int c = 0; c < n_chunks && c < stages; ++c) issue_a(c);

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // RMSNORM: the operand is bfloat16(x * w); the row's 1/rms is applied to the sums at the end (the
    // product is linear in it), so x is read once and its squares are summed on the way
    float ssq_part[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) ssq_part[j] = 0.f;

    float acc[RT][NT][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[rt][j][0] = acc[rt][j][1] = acc[rt][j][2] = acc[rt][j][3] = 0.f;

    // the activations of this warp's steps of chunk c (a chunk has at most LF_WARPS * LF_UNROLL(NT) steps)
    auto load_a = [&](int c, uint4 (&a)[LF_UNROLL(NT)][NT]) {
        const int k0 = c * chunk, cols = min(chunk, K - k0);
#pragma unroll
        for (int u = 0; u < LF_UNROLL(NT); ++u) {
            const int col = (((warp - k0 / 32) & (LF_WARPS - 1)) + u * LF_WARPS) * 32 + t * 8, k = k_begin + k0 + col;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int m = j * 8 + g;
                a[u][j] = zero;
                if (c < n_chunks && m < M && col < cols) {
                    if (PRO == LF_RMSNORM) {
                        const float4 x0 = *reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k);
                        const float4 x1 = *reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k + 4);
                        ssq_part[j] += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w +
                                       x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
                        float w8[8];
                        if (p.norm_w_dtype == PE_BF16) {
                            const uint4 wv = *reinterpret_cast<const uint4*>((const bf16*)p.norm_w + k);
                            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(w2[e]); w8[2 * e] = f.x; w8[2 * e + 1] = f.y; }
                        } else {
                            const float4 w0 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k);
                            const float4 w1 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k + 4);
                            w8[0] = w0.x; w8[1] = w0.y; w8[2] = w0.z; w8[3] = w0.w; w8[4] = w1.x; w8[5] = w1.y; w8[6] = w1.z; w8[7] = w1.w;
                        }
                        a[u][j].x = lf_pack(x0.x * w8[0], x0.y * w8[1]);
                        a[u][j].y = lf_pack(x0.z * w8[2], x0.w * w8[3]);
                        a[u][j].z = lf_pack(x1.x * w8[4], x1.y * w8[5]);
                        a[u][j].w = lf_pack(x1.z * w8[6], x1.w * w8[7]);
                    } else {
                        a[u][j] = lf_ld16(p.A + (size_t)m * p.K + k);
                    }
                }
            }
        }
    };

    uint4 a_cur[LF_UNROLL(NT)][NT], a_next[LF_UNROLL(NT)][NT];
    if (PRO == LF_RMSNORM) load_a(0, a_cur);
    for (int c = 0; c < n_chunks; ++c) {
        const int k0 = c * chunk, cols = min(chunk, K - k0), steps = (cols + 31) / 32;
        const unsigned stage = smem0 + (c % stages) * stage_bytes;
        if (PRO == LF_RMSNORM) load_a(c + 1, a_next);        // in flight while this chunk's W is awaited and used
        const unsigned parity = (unsigned)(c / stages) & 1u;
        const int first = (warp - k0 / 32) & (LF_WARPS - 1);     // this warp's k steps: those of the range that are = warp mod 8,
        if (first < steps && !(lf_bar_wait(bar0 + 8u * (c % stages), parity) &&
                              (PRO != LF_PLAIN || lf_bar_wait(bar_a0 + 8u * (c % stages), parity)))) {
            atomicExch(status, 1);                           // the copies did not arrive: give up, loudly
            return;
        }
#pragma unroll
        for (int u = 0; u < LF_UNROLL(NT); ++u) {
            const int step = first + u * LF_WARPS, col = step * 32 + t * 8;   // however the range is cut into chunks (the sums do not depend on the cut)
            if (step < steps) {                              // the same for all lanes of the warp: the MMA needs them all
                const bool in = col < cols;                  // a last step may be narrower than 32 columns
                uint4 wa[RT], wb[RT];
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    wa[rt] = in ? lf_lds16(stage + (rt * 16 + g) * row_bytes + col * 2) : zero;
                    wb[rt] = (in && tile_rows >= 16) ? lf_lds16(stage + (rt * 16 + 8 + g) * row_bytes + col * 2) : zero;
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4 a = PRO == LF_PLAIN ? (in ? lf_lds16(stage + (tile_rows + j * 8 + g) * row_bytes + col * 2) : zero)
                                                    : a_cur[u][j];
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt) {
                        lf_mma(acc[rt][j], wa[rt].x, wb[rt].x, wa[rt].y, wb[rt].y, a.x, a.y);
                        lf_mma(acc[rt][j], wa[rt].z, wb[rt].z, wa[rt].w, wb[rt].w, a.z, a.w);
                    }
                }
            }
        }
        if (PRO == LF_RMSNORM) {
#pragma unroll
            for (int u = 0; u < LF_UNROLL(NT); ++u)
#pragma unroll
                for (int j = 0; j < NT; ++j) a_cur[u][j] = a_next[u][j];
        }
        if (c + stages < n_chunks) {                         // the stage is free again: refill it
            __syncthreads();
            issue(c + stages);
            if (PRO == LF_PLAIN) issue_a(c + stages);
        }
    }

    // acc[rt][j][e] of lane (g, t): MMA row g (+8 if e & 2) of tile rt, sequence j*8 + 2t + (e & 1)
    if (RED_IN_RING) __syncthreads();                        // every warp has read what it needs of the stages
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[warp][(rt * NT + j) * 4 + e][lane] = acc[rt][j][e];
    if (PRO == LF_RMSNORM) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {                       // lanes (g, 0..3) hold parts of row j*8 + g
            float v = ssq_part[j];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) ssq[warp][j * 8 + g] = v;
        }
    }
    __syncthreads();

    // one thread per (sequence, row of the tile's first group); it sums both groups over the warps
    if (ksplit > 1) lf_cluster_wait();                       // every CTA of the cluster has set up its barrier
    for (int idx = threadIdx.x; idx < RT * NT * 64; idx += 32 * LF_WARPS) {
        const int rt = idx / (NT * 64), j = (idx >> 6) % NT, e1 = (idx >> 5) & 1, ln = idx & 31;
        const int r = ln >> 2, m = j * 8 + 2 * (ln & 3) + e1;
        if (m >= M) continue;
        float v_lo = 0.f, v_hi = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < LF_WARPS; ++w) { v_lo += red[w][(rt * NT + j) * 4 + e1][ln]; v_hi += red[w][(rt * NT + j) * 4 + 2 + e1][ln]; }
        if (PRO == LF_RMSNORM) {
#pragma unroll
            for (int w = 0; w < LF_WARPS; ++w) sum += ssq[w][m];
        }
        if (ksplit > 1) {
            if (ks != 0) {                                   // this range's sums go to the CTA of the first range
                const unsigned at = lf_smem_addr(gather + ((size_t)(ks - 1) * NT * 64 + idx) * 3);
                lf_send(at, v_lo, bar_x0, 0u); lf_send(at + 4u, v_hi, bar_x0, 0u); lf_send(at + 8u, sum, bar_x0, 0u);
                continue;
            }
            if (!lf_bar_wait(bar_x0, 0u)) { atomicExch(status, 2); continue; }
            for (int o = 0; o < ksplit - 1; ++o) {           // in the order of the ranges
                const float* g3 = gather + ((size_t)o * NT * 64 + idx) * 3;
                v_lo += g3[0]; v_hi += g3[1]; sum += g3[2];
            }
        }
        if (PRO == LF_RMSNORM) {
            const float rstd = 1.0f / sqrtf(sum / (float)p.K + p.eps);
            v_lo *= rstd; v_hi *= rstd;
        }

        if (EPI == LF_SWIGLU) {
            const int i = blockIdx.x * 8 * RT + rt * 8 + r;
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
            const int pos = ep_pos;                          // loaded before the main loop (this thread's own m and d)
            if (head < p.n_q + p.n_kv && p.cos_t) {
                const float a = v_lo * ep_cos - v_hi * ep_sin, b = v_lo * ep_sin + v_hi * ep_cos;
                v_lo = a; v_hi = b;
            }
            const bf16 o_lo = __float2bfloat16_rn(v_lo), o_hi = __float2bfloat16_rn(v_hi);
            if (head < p.n_q) {
                bf16* q = (bf16*)p.out + (size_t)m * p.n_q * p.hd + (size_t)head * p.hd;
                q[d] = o_lo; q[d + half] = o_hi;
            } else if (p.store) {
                const int page = ep_page;
                if (page >= 0) {
                    const bool is_k = head < p.n_q + p.n_kv;
                    const int kvh = head - p.n_q - (is_k ? 0 : p.n_kv);
                    bf16* dst = (is_k ? p.k_pool : p.v_pool) +
                                (((size_t)page * p.n_kv + kvh) * PE_PAGE + (pos % PE_PAGE)) * p.hd;
                    dst[d] = o_lo; dst[d + half] = o_hi;
                }
            }
        } else {
            const int n_lo = tile * p.rows * RT + rt * 16 + r, n_hi = n_lo + 8;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int n = h ? n_hi : n_lo;
                if (n >= p.N || (h && p.rows != 16)) continue;
                float v = h ? v_hi : v_lo;
                if (p.bias) v += load_as_f(p.bias, p.bias_dtype, n);
                const size_t o = (size_t)m * p.N + n;
                if (EPI == LF_STORE_F32) ((float*)p.out)[o] = v;
                else if (EPI == LF_STORE_BF16) ((bf16*)p.out)[o] = __float2bfloat16_rn(v);
                else atomicAdd((float*)p.out + o, v);     // the only sum into this element: a reduction in memory, no read to wait for
            }
        }
    }
}

template <int NT, int RT, int PRO, int EPI, bool SPLIT>
static int lf_launch_nt(const LfArgs& a, int tiles, size_t smem, int* status, cudaStream_t s) {
    static size_t allowed = 0;                               // per instantiation: dynamic shared memory that may be asked for
    if (allowed == 0) {                                      // (without opting in: 48 KB less the kernel's static arrays)
        cudaFuncAttributes fa;
        PE_TRY(cudaFuncGetAttributes(&fa, linear_fused_kernel<NT, RT, PRO, EPI, SPLIT>));
        allowed = 48 * 1024 - fa.sharedSizeBytes;
    }
    if (smem > allowed) {
        PE_TRY(cudaFuncSetAttribute(linear_fused_kernel<NT, RT, PRO, EPI, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        allowed = smem;
    }
    if (SPLIT) PE_TRY(pe_launch_cluster(linear_fused_kernel<NT, RT, PRO, EPI, SPLIT>, tiles * a.ksplit, 32 * LF_WARPS, smem, s, (unsigned)a.ksplit, a, status));
    else PE_TRY(pe_launch(linear_fused_kernel<NT, RT, PRO, EPI, SPLIT>, (tiles + RT - 1) / RT, 32 * LF_WARPS, smem, s, a, status));
    return 0;
}

// For a K of several chunks: kilobytes of a stage and of all stages of a CTA (tuning knobs; 0: one CTA an SM
// with chunks of up to 1024 columns).
static int& lf_stage_kb() { static int kb = 48; return kb; }      // measured at the 7B shape: 2 stages of 48 KB, 2 CTAs an SM
static int& lf_budget_kb() { static int kb = 108; return kb; }     // (3.4 TB/s against 2.4 TB/s with one CTA an SM and 58 KB stages)
extern "C" void pe_linear_fused_set_stage_policy(int stage_kb, int budget_kb) { lf_stage_kb() = stage_kb; lf_budget_kb() = budget_kb; }

// Whether products with many tiles take two 16-row tiles a CTA (a tuning knob).
static int& lf_two_tiles() { static int on = 1; return on; }
extern "C" void pe_linear_fused_set_two_tiles(int on) { lf_two_tiles() = on ? 1 : 0; }

// The most ranges of K a tile is cut into (a tuning knob: 1 = never, up to 8).
static int& lf_ksplit_limit() { static int limit = 8; return limit; }
extern "C" void pe_linear_fused_set_max_ksplit(int n) { lf_ksplit_limit() = n < 1 ? 1 : (n > 8 ? 8 : n); }

template <int PRO, int EPI>
static int lf_launch(LfArgs& a, int tiles, int* status, cudaStream_t s) {
    if (!status) return PE_ERR_UNSUPPORTED;
    // A long K with few tiles (fewer CTAs than the GPU has SMs): cut K into ranges, one CTA each, up to
    // 8 to a cluster, while the grid stays within two to three CTAs an SM.
    a.ksplit = 1;
    if (EPI != LF_SWIGLU && EPI != LF_ROPE && a.K > LF_MAX_CHUNK) {
        int want = (a.K + LF_MAX_CHUNK - 1) / LF_MAX_CHUNK;
        if (want > lf_ksplit_limit()) want = lf_ksplit_limit();
        while (want > 1 && (long long)tiles * want * 2 > 5 * 148) --want;     // measured: about 2.3 CTAs an SM is best
        a.ksplit = want;
    }
    a.kc = a.ksplit > 1 ? ((a.K + a.ksplit - 1) / a.ksplit + 31) / 32 * 32 : a.K;
    const int nt = a.M <= 8 ? 1 : 2;
    // Two 16-row tiles a CTA where a product has so many tiles that the activations, which every CTA reads
    // again, would cost as much as the weights (gate and up, the vocabulary), and enough CTAs remain.
    constexpr bool can_two = EPI == LF_SWIGLU || EPI == LF_STORE_F32;
    const bool two = can_two && a.ksplit == 1 && (EPI == LF_SWIGLU || a.rows == 16) && tiles >= 2 * 148 && lf_two_tiles();
    const int tile_rows = two ? 32 : ((EPI == LF_SWIGLU || EPI == LF_ROPE || a.rows == 16) ? 16 : 8);
    const int rows_total = tile_rows + (PRO == LF_PLAIN ? nt * 8 : 0);
    // Chunks of equal length (a short last chunk costs a whole turn of the pipeline).  A range of K that fits
    // one chunk is one chunk.  A longer one is cut so that a stage is about lf_stage_kb() and a CTA holds about
    // lf_budget_kb(): several CTAs then share an SM and stream while another starts up or runs its epilogue.
    const int max_chunk = LF_WARPS * LF_UNROLL(nt) * 32;
    int cap = max_chunk;
    size_t budget = 160u << 10;
    if (a.kc > LF_MAX_CHUNK && lf_stage_kb() > 0) {
        cap = ((lf_stage_kb() << 10) / (rows_total * 2) - LF_ROW_PAD) / 32 * 32;
        if (cap < 128) cap = 128;
        if (cap > max_chunk) cap = max_chunk;
        budget = (size_t)lf_budget_kb() << 10;
    }
    const size_t gather_bytes = (size_t)(a.ksplit - 1) * nt * 64 * 3 * 4;
    const size_t red_all = (size_t)LF_WARPS * (two ? 2 : 1) * nt * 4 * 32 * 4;                   // the warps' partial sums:
    const size_t red_bytes = nt > 1 ? red_all : 0, red_static = nt > 1 ? 0 : red_all;            // in the stages' place, or an array of their own
    auto shape = [&](int cap_, size_t budget_, size_t* ring) {
        const int n_chunks = (a.kc + cap_ - 1) / cap_;
        a.chunk = ((a.kc + n_chunks - 1) / n_chunks + 31) / 32 * 32;
        const size_t stage = (size_t)rows_total * (a.chunk + LF_ROW_PAD) * 2;
        int max_stages = (int)(budget_ / stage);             // chunks in flight: what fits the budget, at most 8
        if (max_stages > 2 * LF_MAX_STAGES) max_stages = 2 * LF_MAX_STAGES;
        if (max_stages < 1) max_stages = 1;
        a.stages = n_chunks < max_stages ? n_chunks : max_stages;
        *ring = (size_t)a.stages * stage > red_bytes ? (size_t)a.stages * stage : red_bytes;
    };
    size_t ring = 0;
    shape(cap, budget, &ring);
    // A grid of two to four CTAs an SM runs as one wave only if that many CTAs fit an SM's 228 KB of shared memory (a
    // CTA's own, 1 KB that the system keeps for it, 1.5 KB of barriers and sums): measured at 9 to 16 rows, where the
    // stages are larger, the down projection's 336 CTAs at two an SM took 14.5 us against 9.6.  Where the shape above
    // does not fit, the stages share what does (two of them at least where K has several chunks).
    const int grid = (two ? (tiles + 1) / 2 : tiles) * a.ksplit, at_once = (grid + 147) / 148;
    if (at_once >= 2 && at_once <= 4) {
        const size_t fits = (size_t)228 * 1024 / at_once - 2560 - gather_bytes - red_static;
        if (ring > fits) {
            const int two_fit = (int)(fits / 2 / (rows_total * 2) - LF_ROW_PAD) / 32 * 32;
            if (two_fit >= 128) shape(two_fit < cap ? two_fit : cap, fits, &ring);
        }
    }
    const size_t smem = ring + gather_bytes;
    constexpr bool can_split = EPI != LF_SWIGLU && EPI != LF_ROPE;
    if (can_split && a.ksplit > 1) {
        if (nt == 1) return lf_launch_nt<1, 1, PRO, EPI, can_split>(a, tiles, smem, status, s);
        return lf_launch_nt<2, 1, PRO, EPI, can_split>(a, tiles, smem, status, s);
    }
    if (can_two && two) {
        if (nt == 1) return lf_launch_nt<1, can_two ? 2 : 1, PRO, EPI, false>(a, tiles, smem, status, s);
        return lf_launch_nt<2, can_two ? 2 : 1, PRO, EPI, false>(a, tiles, smem, status, s);
    }
    if (nt == 1) return lf_launch_nt<1, 1, PRO, EPI, false>(a, tiles, smem, status, s);
    return lf_launch_nt<2, 1, PRO, EPI, false>(a, tiles, smem, status, s);
}

static bool lf_aligned(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// x += a . W^T (+ bias) or out = a . W^T (+ bias); `a` bfloat16 [M <= 16, K], or with `x_norm`
// the float32 rows whose RMSNorm (weights norm_w, eps) is the operand.
// epilogue: 0 store float32, 1 store bfloat16, 2 add into float32 out.
extern "C" int pe_linear_fused(const void* a, const float* x_norm, const void* norm_w, int norm_w_dtype, float eps,
                               const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M, int N,
                               int K, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 || epilogue < 0 || epilogue > 2 || !lf_aligned(W) || !lf_aligned(x_norm ? (const void*)x_norm : a))
        return PE_ERR_UNSUPPORTED;
    LfArgs p = {};
    p.A = (const bf16*)a; p.X = x_norm; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps;
    p.W = (const bf16*)W; p.bias = bias; p.bias_dtype = bias_dtype; p.out = out; p.M = M; p.N = N; p.K = K;
    p.rows = (N + 15) / 16 >= 148 ? 16 : 8;                  // small matrices: more, thinner CTAs
    const int tiles = (N + p.rows - 1) / p.rows;
    cudaStream_t s = (cudaStream_t)stream;
    if (x_norm) {
        if (epilogue == 0) return lf_launch<LF_RMSNORM, LF_STORE_F32>(p, tiles, status, s);
        if (epilogue == 1) return lf_launch<LF_RMSNORM, LF_STORE_BF16>(p, tiles, status, s);
        return lf_launch<LF_RMSNORM, LF_ACCUM>(p, tiles, status, s);
    }
    if (epilogue == 0) return lf_launch<LF_PLAIN, LF_STORE_F32>(p, tiles, status, s);
    if (epilogue == 1) return lf_launch<LF_PLAIN, LF_STORE_BF16>(p, tiles, status, s);
    return lf_launch<LF_PLAIN, LF_ACCUM>(p, tiles, status, s);
}

// act[M, I] = silu(h . Wg^T) * (h . Wu^T), h = RMSNorm(x); W = [Wg; Wu] is [2I, K].
extern "C" int pe_norm_gate_up_swiglu(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* W,
                                      void* act, int M, int I, int K, int* status, void* stream) {
    if (M <= 0 || I <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 || I % 8 || !lf_aligned(W) || !lf_aligned(x)) return PE_ERR_UNSUPPORTED;
    LfArgs p = {};
    p.X = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps; p.W = (const bf16*)W; p.out = act;
    p.M = M; p.N = 2 * I; p.K = K; p.I = I; p.rows = 16;
    return lf_launch<LF_RMSNORM, LF_SWIGLU>(p, I / 8, status, (cudaStream_t)stream);
}

// q[M, n_q * hd] and the cache pages of keys and values from h = RMSNorm(x) (or from bfloat16
// `a` when x is null): project with W = [Wq; Wk; Wv], add bias, rotate q and k by position
// (cos_t null: no rotation), write keys and values at (page of the token's sequence, position).
extern "C" int pe_norm_qkv_rope_store(const void* a, const float* x, const void* norm_w, int norm_w_dtype, float eps,
                                      const void* W, const void* bias, int bias_dtype, void* q_out, int M, int K,
                                      int n_q, int n_kv, int hd, const float* cos_t, const float* sin_t,
                                      const int* tok_pos, const int* tok_row, void* k_pool, void* v_pool,
                                      const int* block_table, int table_stride, int store, int* status, void* stream) {
    if (M <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 || hd % 16 || !lf_aligned(W) || !lf_aligned(x ? (const void*)x : a)) return PE_ERR_UNSUPPORTED;
    LfArgs p = {};
    p.A = (const bf16*)a; p.X = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps;
    p.W = (const bf16*)W; p.bias = bias; p.bias_dtype = bias_dtype; p.out = q_out; p.M = M; p.N = (n_q + 2 * n_kv) * hd;
    p.K = K; p.rows = 16; p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.cos_t = cos_t; p.sin_t = sin_t; p.tok_pos = tok_pos;
    p.tok_row = tok_row; p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.block_table = block_table;
    p.table_stride = table_stride; p.store = store;
    const int tiles = (n_q + 2 * n_kv) * (hd / 16);
    if (x) return lf_launch<LF_RMSNORM, LF_ROPE>(p, tiles, status, (cudaStream_t)stream);
    return lf_launch<LF_PLAIN, LF_ROPE>(p, tiles, status, (cudaStream_t)stream);
}
