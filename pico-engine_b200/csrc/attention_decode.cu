// Attention of single tokens over the paged bfloat16 cache (decoding), compiled for one head
// size (PE_HEAD_DIM, a multiple of 16 up to 256).
//
// Grid: (range of the sequence's pages, kv head x tile of 16 query heads, token); the CTAs of
// the ranges of one (token, kv head) are one thread-block cluster.  All query heads that share
// a kv head sit in the 16 rows of one MMA tile, so keys and values are read once for the
// group.  A page of the cache holds the 64 keys (or values) of one kv head contiguously: a
// producer warp brings whole pages into a ring in shared memory with bulk asynchronous copies
// (cp.async.bulk, completing on an mbarrier), as many pages ahead as the ring holds, so the
// bytes in flight do not depend on registers or on how many warps are resident.  The copies
// start before this kernel waits for the one before it: that kernel can have written only the
// newest token's key and value, and the warp that meets this row fetches it again after the
// wait.  The consumer warps (8 or 16, see below) take 16 keys of a page each:
// scores S = Q.K^T with mma.sync m16n8k16 (16-byte loads from shared memory straight into B
// fragments, the head dimension permuted identically in Q), online softmax in float32 on the
// accumulator registers, then O += P.V where V fragments are transposed in registers with
// movmatrix.  The loop body is kept small: these kernels run for microseconds, each warp
// passes through it a few times, and fetching instructions costs as much as executing them.  The warps of a CTA merge their (max, sum, O) in shared memory; the CTAs of
// a cluster then read one another's results through distributed shared memory, each merging a
// slice of the output in the order of the ranges, so there is no second kernel and no scratch
// in global memory.  How a sequence's pages are dealt to the ranges depends on its own length
// only, never on the other sequences of the batch.
//
// Every wait on an mbarrier is bounded; one that runs out sets *status and the CTA goes on to
// its cluster barriers without computing, so that no CTA of the cluster is left waiting.
//
// pico-engine's counterpart is _decode_attn_fwd (src/pico_engine/kernels.py:90-126): one
// program per query head, looping over the whole buffer.
#ifndef PE_HEAD_DIM
#error "compile with -DPE_HEAD_DIM=<head size>"
#endif
#include "common.cuh"
#include <map>
#include <mutex>
#include <utility>

#define AD_HD PE_HEAD_DIM
#define AD_NCHUNK ((AD_HD + 31) / 32)
// The kernel is compiled for 8 and for 16 consumer warps (one more warp is the producer).  Four warps share a
// page, so 2 or 4 pages are under way at once.  16 warps (one CTA an SM) are quicker where few sequences
// have long contexts; 8 warps (two CTAs an SM for head sizes up to 64) everywhere else.
#define AD_CTAS(WARPS) (((WARPS) == 16 || AD_HD > 64) ? 1 : 2)
#define AD_MAX_STAGES 12                             // pages in flight per CTA
#define AD_MAX_SPLITS 16                             // page ranges of a sequence = CTAs of a cluster (8 is the portable limit)
#define AD_KV_BYTES (PE_PAGE * AD_HD * 2)            // the keys (or the values) of one page and kv head
#define AD_STAGE_BYTES (2 * AD_KV_BYTES)
#define AD_ROW (AD_HD + 2)                           // floats between the rows of a warp's partial sums (skews the banks)
#define AD_RES_BYTES ((16 * (AD_HD + 3 * AD_MAX_SPLITS) * 4 + 127) / 128 * 128)   // what the merge of the ranges gathers
#define AD_SCRATCH_BYTES(WARPS) ((WARPS) * 16 * (AD_ROW + 2) * 4)
#define AD_SMEM_BUDGET(WARPS) ((AD_CTAS(WARPS) == 2 ? 108 : 190) * 1024)   // per CTA; leaves room for the next kernel's first CTAs
#define AD_WAIT_CYCLES 2000000000ll                  // about a second of SM clock

__device__ __forceinline__ unsigned ad_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ad_bar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void ad_bar_expect(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ad_bar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ad_bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// true when the phase with this parity has completed; false when the wait ran out
__device__ __forceinline__ bool ad_bar_test(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0u;
}
__device__ __forceinline__ bool ad_bar_wait(unsigned bar, unsigned parity) {
    if (ad_bar_test(bar, parity)) return true;               // the usual case costs one test
    const long long deadline = clock64() + AD_WAIT_CYCLES;
    for (;;) {
        if (ad_bar_test(bar, parity)) return true;
        if (clock64() > deadline) return false;
        __nanosleep(32);
    }
}
__device__ __forceinline__ void ad_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void ad_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ unsigned ad_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the same shared-memory address in CTA `rank` of the cluster
__device__ __forceinline__ unsigned ad_map(unsigned local_addr, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// a float into another CTA's shared memory; its 4 bytes are counted on that CTA's mbarrier
__device__ __forceinline__ void ad_st_async(unsigned remote_addr, float v, unsigned remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(remote_addr), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ uint4 ad_lds16(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
// Queries were written by the kernel before this one: a plain coherent load, never the read-only path.
__device__ __forceinline__ uint4 ad_ld16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ad_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ad_transpose(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ unsigned ad_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Fragment conventions (lane = 4*g + t).  Scores of a 16-key tile are two m16n8 accumulators
// s[j][e]: row (e & 2 ? g + 8 : g), key j*8 + 2t + (e & 1).  The output accumulators are
// acc[c][r][e]: row as above, head-dimension column c*32 + t*8 + 2r + (e & 1).  Q fragments
// qf[c][0/1] (rows g / g + 8) and the 16-byte loads of key rows hold columns c*32 + t*8 .. +8,
// so both operands of S = Q.K^T see the head dimension in the same permuted order.

__device__ __forceinline__ float ad_ex2(float x) {          // 2^x; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One tile of 16 keys against the warp's 16 query rows.  kt, vt: shared-memory addresses of the
// tile's first key and value row; key0: position of that key.  At least one key of the tile is
// visible (lo <= key <= pos), so every row's running max is finite after it.
__device__ __forceinline__ void ad_consume(float (&acc)[AD_NCHUNK][4][4], float (&m_run)[2], float (&l_run)[2],
                                           const uint4 (&qf)[AD_NCHUNK][2], unsigned kt, unsigned vt, int key0, int lo,
                                           int pos, float scale_log2e, int g, int t) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int c = 0; c < AD_NCHUNK; ++c) {
            const bool cin = c * 32 + t * 8 + 8 <= AD_HD;
            const uint4 kf = cin ? ad_lds16(kt + (unsigned)(((j * 8 + g) * AD_HD + c * 32 + t * 8) * 2)) : zero;
            ad_mma(sc[j], qf[c][0].x, qf[c][1].x, qf[c][0].y, qf[c][1].y, kf.x, kf.y);
            ad_mma(sc[j], qf[c][0].z, qf[c][1].z, qf[c][0].w, qf[c][1].w, kf.z, kf.w);
        }
    }
    // sc[j][e]: row (e & 2 ? g + 8 : g), key key0 + j*8 + 2t + (e & 1)
    if (key0 < lo || key0 + 15 > pos) {                      // a tile on the edge of what is visible
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + j * 8 + 2 * t + (e & 1);
                if (key < lo || key > pos) sc[j][e] = -INFINITY;
            }
    }
    float tmax[2];
#pragma unroll
    for (int r = 0; r < 2; ++r)
        tmax[r] = fmaxf(fmaxf(sc[0][2 * r], sc[0][2 * r + 1]), fmaxf(sc[1][2 * r], sc[1][2 * r + 1])) * scale_log2e;
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
        const float m_new = fmaxf(m_run[r], tmax[r]);
        alpha[r] = ad_ex2(m_run[r] - m_new);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
    }
    float p[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p[j][e] = ad_ex2(fmaf(sc[j][e], scale_log2e, -m_run[e >> 1]));
            l_run[e >> 1] += p[j][e];
        }
    const unsigned pa0 = ad_pack(p[0][0], p[0][1]), pa1 = ad_pack(p[0][2], p[0][3]);
    const unsigned pa2 = ad_pack(p[1][0], p[1][1]), pa3 = ad_pack(p[1][2], p[1][3]);
    // the accumulators are scaled only when some row's max has moved (it seldom does after the first tiles)
    const bool moved = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
#pragma unroll
    for (int c = 0; c < AD_NCHUNK; ++c) {
        const bool cin = c * 32 + t * 8 + 8 <= AD_HD;
        if (moved) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                acc[c][r][0] *= alpha[0]; acc[c][r][1] *= alpha[0];
                acc[c][r][2] *= alpha[1]; acc[c][r][3] *= alpha[1];
            }
        }
        const uint4 v0 = cin ? ad_lds16(vt + (unsigned)((g * AD_HD + c * 32 + t * 8) * 2)) : zero;
        const uint4 v1 = cin ? ad_lds16(vt + (unsigned)(((8 + g) * AD_HD + c * 32 + t * 8) * 2)) : zero;
        const unsigned lo_r[4] = {v0.x, v0.y, v0.z, v0.w}, hi_r[4] = {v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int r = 0; r < 4; ++r)
            ad_mma(acc[c][r], pa0, pa1, pa2, pa3, ad_transpose(lo_r[r]), ad_transpose(hi_r[r]));
    }
}

template <int AD_WARPS>
__global__ void __launch_bounds__(32 * (AD_WARPS + 1), AD_CTAS(AD_WARPS)) attention_decode_kernel(
    const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool,
    const int* block_table, int table_stride, const int* tok_pos,
    const int* tok_row, int nh, int nkv, int window, float scale_log2e, int n_splits, int stages,
    int* status, bf16* out) {
    constexpr int AD_GROUPS = AD_WARPS / 4, AD_THREADS = 32 * (AD_WARPS + 1);
    extern __shared__ __align__(128) unsigned char ad_smem[];   // result rows, then the ring (later: the warps' partial results)
    __shared__ __align__(8) unsigned long long bars[2 * AD_MAX_STAGES + 1];
    __shared__ int page_ok[AD_MAX_STAGES];                      // whether the stage holds a page (written by the producer)
    __shared__ float row_max[16];                               // the CTA's max of every row
    __shared__ int page_list[32];                               // the producer's next entries of the page table
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int tok = blockIdx.z;
    const int split = n_splits > 1 ? (int)ad_cluster_rank() : 0;
    const int G = nh / nkv, head_tiles = (G + 15) / 16;
    const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y % head_tiles;
    // positions and page tables were uploaded before the step began: they may be read before the wait
    const int pos = tok_pos[tok];
    const int* table = block_table + (size_t)tok_row[tok] * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_page = lo / PE_PAGE, last_page = pos / PE_PAGE;
    const int per_split = (last_page - first_page + n_splits) / n_splits;          // ceil(pages / n_splits)
    const int p0 = first_page + split * per_split;
    int n_mine = max(0, min(p0 + per_split, last_page + 1) - p0);
    if (n_mine > stages && stages % AD_GROUPS) {             // a ring the host must not give (see how the warps share the pages)
        if (threadIdx.x == 0) atomicExch(status, 3);
        n_mine = 0;
    }

    // The merge of the ranges: the head dimension is dealt to the CTAs of the cluster in slices of `slice`
    // columns.  gather[range][row][0..slice) holds that range's sums for this CTA's columns, [slice] the
    // row's max and [slice + 1] its sum; the other CTAs write theirs with st.async, which counts bytes on gbar.
    float* gather = reinterpret_cast<float*>(ad_smem);
    unsigned char* ring = ad_smem + AD_RES_BYTES;
    const unsigned ring0 = ad_smem_addr(ring), full0 = ad_smem_addr(bars), empty0 = full0 + 8u * AD_MAX_STAGES;
    const unsigned gather0 = ad_smem_addr(gather), gbar = empty0 + 8u * AD_MAX_STAGES;
    const int rows = min(16, G - ht * 16);
    const int slice = (AD_HD + n_splits - 1) / n_splits, grow = slice + 2;
    const int my_cols = max(0, min(slice, AD_HD - split * slice));

    // Four warps share a page, AD_GROUPS pages are under way: warp w takes keys (w % 4) * 16 .. +16 of the
    // pages i with i % AD_GROUPS == w / 4.  A ring that wraps must give every stage to the same warps each
    // time round: a wait by parity tells a phase only from its neighbours, so a warp has to see every
    // phase of a barrier that it waits on.  The host sizes the ring so.
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { ad_bar_init(full0 + 8u * s, 1u); ad_bar_init(empty0 + 8u * s, 4u); }
        ad_bar_init(gbar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (n_splits > 1) ad_bar_expect(gbar, my_cols > 0 ? (unsigned)((n_splits - 1) * rows * (my_cols + 2) * 4) : 0u);
    }
    __syncthreads();
    if (n_splits > 1) ad_cluster_arrive();                   // waited for just before the first write to another CTA

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[AD_NCHUNK][4][4];
#pragma unroll
    for (int c = 0; c < AD_NCHUNK; ++c)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[c][r][0] = acc[c][r][1] = acc[c][r][2] = acc[c][r][3] = 0.f;

    if (warp == AD_WARPS) {
        // ---- the producer: page i of this range into stage i % stages.  The warp reads 32 entries of the
        // page table at a time; lane 0 then waits for each stage to be free and issues the copies.  It does
        // not wait for the preceding kernel: see the consumers on the one row that kernel may be writing.
        bool alive = true;
        for (int base = 0; base < n_mine && alive; base += 32) {
            __syncwarp();
            if (base + lane < n_mine) page_list[lane] = table[p0 + base + lane];
            __syncwarp();
            if (lane == 0) {
                int s = base % stages, round = base / stages;
                for (int i = base; i < min(base + 32, n_mine); ++i) {
                    if (round > 0 && !ad_bar_wait(empty0 + 8u * s, (unsigned)(round - 1) & 1u)) {
                        atomicExch(status, 2);
                        alive = false;
                        break;
                    }
                    const int page = page_list[i - base];
                    page_ok[s] = page >= 0;
                    if (page < 0) {                              // a page the window has left behind: nothing to copy
                        ad_bar_arrive(full0 + 8u * s);
                    } else {
                        const size_t off = ((size_t)page * nkv + kvh) * (size_t)(PE_PAGE * AD_HD);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the stage's readers precede its refill
                        ad_bar_expect(full0 + 8u * s, AD_STAGE_BYTES);
                        ad_bulk_copy(ring0 + s * AD_STAGE_BYTES, k_pool + off, AD_KV_BYTES, full0 + 8u * s);
                        ad_bulk_copy(ring0 + s * AD_STAGE_BYTES + AD_KV_BYTES, v_pool + off, AD_KV_BYTES, full0 + 8u * s);
                    }
                    if (++s == stages) { s = 0; ++round; }
                }
            }
            alive = __shfl_sync(0xffffffffu, alive, 0);
        }
    } else {
        // ---- the consumers
        const int last_phys = table[last_page];               // the page of the newest token
        pdl_wait();
        const int r_lo = ht * 16 + g, r_hi = r_lo + 8;        // this lane's two query heads within the group
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        uint4 qf[AD_NCHUNK][2];
#pragma unroll
        for (int c = 0; c < AD_NCHUNK; ++c) {
            const int col = c * 32 + t * 8;
            const bool cin = col + 8 <= AD_HD;
            const bf16* qp = q + (size_t)tok * q_stride + col;
            qf[c][0] = (cin && r_lo < G) ? ad_ld16(qp + (size_t)(kvh * G + r_lo) * AD_HD) : zero;
            qf[c][1] = (cin && r_hi < G) ? ad_ld16(qp + (size_t)(kvh * G + r_hi) * AD_HD) : zero;
        }
        const int grp = warp >> 2, first_key = (warp & 3) * 16;
        const bool wraps = n_mine > stages;
        bool dead = false;
        int s = grp % stages, round = grp / stages;
        for (int i = grp; i < n_mine; i += AD_GROUPS) {
            if (!dead && !__all_sync(0xffffffffu, ad_bar_wait(full0 + 8u * s, (unsigned)round & 1u))) {
                dead = true;
                if (lane == 0) atomicExch(status, 1);
            }
            const int key0 = (p0 + i) * PE_PAGE + first_key;
            if (!dead && key0 <= pos && key0 + 16 > lo && page_ok[s]) {
                const unsigned kt = ring0 + s * AD_STAGE_BYTES + (unsigned)(first_key * AD_HD * 2), vt = kt + AD_KV_BYTES;
                if (pos < key0 + 16) {
                    // The newest token's row: the page was copied while the kernel that writes this row may still
                    // have been running, so it is fetched again now, after the wait for that kernel.
                    const size_t off = (((size_t)last_phys * nkv + kvh) * PE_PAGE + (pos % PE_PAGE)) * AD_HD;
                    const unsigned at = (unsigned)(((pos - key0) * AD_HD + lane * 8) * 2);
                    if (lane * 8 < AD_HD) {
                        const uint4 kr = ad_ld16(k_pool + off + lane * 8), vr = ad_ld16(v_pool + off + lane * 8);
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(kt + at), "r"(kr.x), "r"(kr.y), "r"(kr.z), "r"(kr.w) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(vt + at), "r"(vr.x), "r"(vr.y), "r"(vr.z), "r"(vr.w) : "memory");
                    }
                    __syncwarp();
                }
                ad_consume(acc, m_run, l_run, qf, kt, vt, key0, lo, pos, scale_log2e, g, t);
            }
            if (wraps) {                                     // a stage that is used again: tell the producer it is free
                __syncwarp();
                if (lane == 0) ad_bar_arrive(empty0 + 8u * s);
            }
            s += AD_GROUPS;
            while (s >= stages) { s -= stages; ++round; }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        }
    }

    // ---- merge the warps: the ring is free once every warp has left its loop.  Each warp scales its sums
    // to the CTA's max of the row first, so that merging is adding.
    __syncthreads();
    float* part = reinterpret_cast<float*>(ring);           // [AD_WARPS][16][AD_ROW] sums, then per (warp, row): max, sum
    float* w_max = part + AD_WARPS * 16 * AD_ROW;
    float* w_sum = w_max + AD_WARPS * 16;
    if (warp < AD_WARPS && t == 0) { w_max[warp * 16 + g] = m_run[0]; w_max[warp * 16 + g + 8] = m_run[1]; }
    __syncthreads();
    if (warp < AD_WARPS) {
        float scale[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) m = fmaxf(m, w_max[w * 16 + g + 8 * r]);
            scale[r] = m_run[r] == -INFINITY ? 0.f : ad_ex2(m_run[r] - m);
            if (t == 0) w_sum[warp * 16 + g + 8 * r] = l_run[r] * scale[r];
            if (warp == 0 && t == 0) row_max[g + 8 * r] = m;
        }
        float* mine = part + (size_t)warp * 16 * AD_ROW;
#pragma unroll
        for (int c = 0; c < AD_NCHUNK; ++c)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int col = c * 32 + t * 8 + 2 * r;       // acc[c][r][0..1]: row g, cols col, col+1; [2..3]: row g+8
                if (col < AD_HD) {
                    *reinterpret_cast<float2*>(mine + g * AD_ROW + col) = make_float2(acc[c][r][0] * scale[0], acc[c][r][1] * scale[0]);
                    *reinterpret_cast<float2*>(mine + (g + 8) * AD_ROW + col) = make_float2(acc[c][r][2] * scale[1], acc[c][r][3] * scale[1]);
                }
            }
    }
    __syncthreads();
    if (n_splits > 1) ad_cluster_wait();                     // every CTA of the cluster has set up its barrier
    for (int idx = threadIdx.x; idx < rows * AD_HD; idx += AD_THREADS) {
        const int row = idx / AD_HD, col = idx % AD_HD;
        const float m = row_max[row];
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            o += part[((size_t)w * 16 + row) * AD_ROW + col];
            l += w_sum[w * 16 + row];
        }
        if (n_splits == 1) {
            out[((size_t)tok * nh + kvh * G + ht * 16 + row) * AD_HD + col] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
            continue;
        }
        // the CTA that owns this column gets the sum; every CTA that owns columns gets the row's max and sum
        const int dst = col / slice, j = col - dst * slice;
        const unsigned at = gather0 + (unsigned)(((split * 16 + row) * grow + j) * 4);
        if (dst == split) gather[(split * 16 + row) * grow + j] = o;
        else ad_st_async(ad_map(at, (unsigned)dst), o, ad_map(gbar, (unsigned)dst));
        if (col * slice < AD_HD) {                           // thread `col` of the row tells CTA `col` the row's max and sum
            const int d = col;
            const unsigned at_m = gather0 + (unsigned)(((split * 16 + row) * grow + slice) * 4);
            if (d == split) {
                gather[(split * 16 + row) * grow + slice] = m; gather[(split * 16 + row) * grow + slice + 1] = l;
            } else {
                ad_st_async(ad_map(at_m, (unsigned)d), m, ad_map(gbar, (unsigned)d));
                ad_st_async(ad_map(at_m + 4u, (unsigned)d), l, ad_map(gbar, (unsigned)d));
            }
        }
    }
    if (n_splits == 1) return;

    // ---- merge the ranges: this CTA's columns of every range's result have been sent here
    __syncthreads();
    if (!ad_bar_wait(gbar, 0u)) {
        if (threadIdx.x == 0) atomicExch(status, 4);
        return;
    }
    for (int idx = threadIdx.x; idx < rows * my_cols; idx += AD_THREADS) {
        const int row = idx / my_cols, j = idx - row * my_cols;
        float m = -INFINITY;
        for (int r = 0; r < n_splits; ++r) m = fmaxf(m, gather[(r * 16 + row) * grow + slice]);
        float o = 0.f, l = 0.f;
        for (int r = 0; r < n_splits; ++r) {
            const float* src = gather + (r * 16 + row) * grow;
            const float wgt = (src[slice] == -INFINITY) ? 0.f : exp2f(src[slice] - m);
            o = fmaf(src[j], wgt, o);
            l = fmaf(src[slice + 1], wgt, l);
        }
        out[((size_t)tok * nh + kvh * G + ht * 16 + row) * AD_HD + split * slice + j] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

extern "C" int pe_attention_decode_head_dim() { return AD_HD; }
extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }

// The host side of one variant of the kernel.  In an unnamed namespace: the libraries of several head sizes
// live in one process, and the function-local statics of a template with external linkage would be one
// object for all of them (the dynamic linker makes such symbols unique across libraries).
namespace {
template <int WARPS>
struct AdVariant {
    static constexpr int threads = 32 * (WARPS + 1), groups = WARPS / 4, ctas_per_sm = AD_CTAS(WARPS);

    static size_t smem_bytes(int stages) {
        size_t body = (size_t)stages * AD_STAGE_BYTES;
        if (body < (size_t)AD_SCRATCH_BYTES(WARPS)) body = AD_SCRATCH_BYTES(WARPS);
        return AD_RES_BYTES + body;
    }

    static int allow_smem(size_t smem) {
        static size_t allowed = 48 * 1024 - 512;
        static bool wide = false;
        if (!wide) {                                         // clusters of more than 8 CTAs are an opt-in; if it is refused,
            cudaFuncSetAttribute(attention_decode_kernel<WARPS>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);   // the
            cudaGetLastError();                              // occupancy query below answers 0 for them and fewer ranges are used
            wide = true;
        }
        if (smem > allowed) {
            PE_TRY(cudaFuncSetAttribute(attention_decode_kernel<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            allowed = smem;
        }
        return 0;
    }

    // How many clusters of `splits` CTAs with this much shared memory the GPU holds at once (a
    // cluster needs its SMs in one GPC, so this is less than SMs x CTAs per SM / splits); 0 on error.
    static int clusters_at_once(int splits, size_t smem) {
        static std::mutex lock;
        static std::map<std::pair<int, size_t>, int> known;
        std::lock_guard<std::mutex> hold(lock);
        auto it = known.find({splits, smem});
        if (it != known.end()) return it->second;
        int n = 0;
        if (allow_smem(smem) == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(splits, 1, 148 * ctas_per_sm);
            cfg.blockDim = dim3(threads);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<WARPS>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        }
        known[{splits, smem}] = n;
        return n;
    }

    // The launch shape for `ctas` (token, kv head, head tile) triples over at most `pages` pages each: how many
    // page ranges a sequence is cut into and how many pages a CTA keeps in flight.  As many ranges as fill the
    // GPU once, and no more than let all clusters be resident at the same time.
    static int shape(int ctas, int pages, int limit, int* stages_out) {
        const int fit = (AD_SMEM_BUDGET(WARPS) - AD_RES_BYTES) / AD_STAGE_BYTES;
        int splits = 148 * ctas_per_sm / ctas;
        if (splits > limit) splits = limit;
        if (splits > pages) splits = pages;
        if (splits < 1) splits = 1;
        int stages = 1;
        for (;; --splits) {
            const int most = (pages + splits - 1) / splits;  // pages of a CTA's range
            stages = most;
            if (stages > fit) stages = fit;
            if (stages > AD_MAX_STAGES) stages = AD_MAX_STAGES;
            // A ring that is used more than once has a multiple of `groups` stages: a stage then always serves
            // the same warps, which therefore see every phase of its barriers (see the kernel).
            if (stages < most) stages -= stages % groups;
            if (splits == 1 || stages < 1 || clusters_at_once(splits, smem_bytes(stages)) >= ctas) break;
        }
        *stages_out = stages;
        return splits;
    }

    static int launch(dim3 grid, int n_splits, int stages, cudaStream_t stream, const bf16* q, int q_stride, const bf16* k_pool,
                      const bf16* v_pool, const int* block_table, int table_stride, const int* tok_pos, const int* tok_row,
                      int nh, int nkv, int window, float scale_log2e, int* status, bf16* out, bool early) {
        const size_t smem = smem_bytes(stages);
        { const int e = allow_smem(smem); if (e) return e; }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        int n_attr = 0;
        if (pe_pdl_enabled() && early) {                   // without it the kernel starts when all work before it in the stream has ended
            attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
            ++n_attr;
        }
        if (n_splits > 1) {
            attr[n_attr].id = cudaLaunchAttributeClusterDimension;
            attr[n_attr].val.clusterDim.x = n_splits; attr[n_attr].val.clusterDim.y = 1; attr[n_attr].val.clusterDim.z = 1;
            ++n_attr;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        PE_TRY(cudaLaunchKernelEx(&cfg, attention_decode_kernel<WARPS>, q, q_stride, k_pool, v_pool, block_table, table_stride,
                                  tok_pos, tok_row, nh, nkv, window, scale_log2e, n_splits, stages, status, out));
        PE_LAUNCH_CHECK();
        return 0;
    }
};
}  // namespace

// The most page ranges a sequence is cut into (a tuning knob: 1 .. AD_MAX_SPLITS).
static int& ad_split_limit() { static int limit = AD_MAX_SPLITS; return limit; }
extern "C" void pe_attention_decode_set_max_splits(int n) { ad_split_limit() = n < 1 ? 1 : (n > AD_MAX_SPLITS ? AD_MAX_SPLITS : n); }

// Which variant and shape a launch takes: a function of the launch's sizes (and of the GPU) only, never of
// the sequences' lengths: the same launch is replayed as sequences grow.  Measured at head size 64: 16 warps
// win where at most 32 CTA-triples have 8 or more pages each (8 sequences of 4,096 tokens: 8.1 us against
// 8.3 us), 8 warps elsewhere (1 sequence: 4.9 us against 5.3 us; 64 sequences: 24 us against 27 us).
static bool ad_choose(int T, int nh, int nkv, int max_context, int* splits_out, int* stages_out) {
    const int G = nh / nkv, ctas = T * nkv * ((G + 15) / 16);
    const int pages = (max_context + PE_PAGE - 1) / PE_PAGE;
    if constexpr (AD_HD <= 64) {                             // larger heads need the registers: 8 warps only
        if (ctas <= 32) {
            int stages = 0;
            const int splits = AdVariant<16>::shape(ctas, pages, ad_split_limit(), &stages);
            if ((pages + splits - 1) / splits >= 8) { *splits_out = splits; *stages_out = stages; return true; }
        }
    }
    *splits_out = AdVariant<8>::shape(ctas, pages, ad_split_limit(), stages_out);
    return false;
}

extern "C" int pe_attention_decode_splits(int T, int nh, int nkv, int max_context, int* stages_out) {
    int splits = 1, stages = 1;
    ad_choose(T, nh, nkv, max_context, &splits, &stages);
    if (stages_out) *stages_out = stages;
    return splits;
}

extern "C" int pe_attention_decode(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                   const int* block_table, int table_stride, const int* tok_pos, const int* tok_row,
                                   int T, int nh, int nkv, int hd, int window, float scale, int max_context,
                                   int early_pages, int* status, void* stream) {
    // early_pages 1: the kernel may start while the kernels before it in the stream still run, and copies cache pages
    // at once; those kernels (the one before it, and the one before that, which it can overlap too) must then have
    // written no cache row but each token's own (which is fetched again after the wait).  0: it starts when they have ended.
    if (T <= 0) return 0;
    if (hd != AD_HD || nkv <= 0 || nh % nkv || max_context <= 0 || q_stride % 8 || T > 65535 || !status) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return PE_ERR_UNSUPPORTED;
    const int G = nh / nkv;
    if ((long long)nkv * ((G + 15) / 16) > 65535) return PE_ERR_UNSUPPORTED;
    int n_splits = 1, stages = 0;
    const bool wide = ad_choose(T, nh, nkv, max_context, &n_splits, &stages);
    if (stages < 1) return PE_ERR_UNSUPPORTED;
    const dim3 grid(n_splits, nkv * ((G + 15) / 16), T);
    const float scale_log2e = scale * 1.4426950408889634f;
    if constexpr (AD_HD <= 64) {
        if (wide)
            return AdVariant<16>::launch(grid, n_splits, stages, (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_pool,
                                         (const bf16*)v_pool, block_table, table_stride, tok_pos, tok_row, nh, nkv, window,
                                         scale_log2e, status, (bf16*)out, early_pages != 0);
    }
    return AdVariant<8>::launch(grid, n_splits, stages, (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_pool,
                                (const bf16*)v_pool, block_table, table_stride, tok_pos, tok_row, nh, nkv, window, scale_log2e,
                                status, (bf16*)out, early_pages != 0);
}
