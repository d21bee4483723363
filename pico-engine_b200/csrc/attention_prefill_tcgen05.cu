// Causal attention of many tokens per sequence over the paged bfloat16 cache on the
// 5th-generation tensor cores, for head sizes 64 and 128 (PE_HEAD_DIM): both products of flash
// attention run as tcgen05.mma with their accumulators in tensor memory.
//
//   one CTA   = a run of up to 128 consecutive tokens of one sequence x one query head
//   a step    = two pages of the cache (128 keys): products this small cost the tensor core more in
//               fixed latency than in work, so fewer and larger ones are issued
//   warp 0      loader: TMA tiled loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the run's
//               queries and, step after step, of the pages' keys and values into a ring; it alone
//               reads the page table and tells the others through flags which pages are there
//   warp 1      allocates tensor memory; one lane issues S = Q.K^T (128 x 128, K = head size) into
//               one of two S buffers and O += P.V (128 x head size, K = 128 keys): S of the next
//               step is issued before P.V of this one, so the softmax never waits for the product
//   warps 2-9   softmax, two threads a query row, one for each page of the step: tcgen05.ld of its
//               64 scores, mask, maximum (the two tell each other theirs through shared memory),
//               P = 2^(s - max) rounded to bfloat16 into one of two swizzled shared-memory tiles,
//               the A operand of P.V, and the row sum in float32; when a row's reference point
//               moves, the row of O in tensor memory is rescaled (tcgen05.ld / tcgen05.st), each
//               thread its half, before P.V runs.  Two warps on each of the SM's four schedulers
//               hide each other's latencies; the exponentials (one special-function unit a
//               scheduler) and the tensor core's time for the two products then bound a step.
//
// Values lie in the cache as [key][head size], which is the MN-major form of the B operand of
// P.V: its shared-memory descriptor steps 8 keys by 1024 bytes and 64 columns by one panel.
// Every mbarrier wait is bounded by the clock; a wait that runs out sets *status to 5, the roles
// leave their loops, tensor memory is freed and the CTA returns.
//
// pico-engine hands this to torch's fused attention after copying keys and values out of the
// cache (src/pico_engine/model.py:201-209).
#ifndef PE_HEAD_DIM
#error "compile with -DPE_HEAD_DIM=<head size>"
#endif
#include "common.cuh"
#include <cuda.h>

#if PE_HEAD_DIM == 64 || PE_HEAD_DIM == 128

#define AT_HD PE_HEAD_DIM
#define AT_QTILE 128
#define AT_KTILE PE_PAGE
#define AT_PANELS (AT_HD / 64)                     // 64-column panels of a row: one 128-byte swizzle atom each
#define AT_STAGES (AT_HD == 64 ? 3 : 2)            // steps in flight or in use; a step is two pages (128 keys)
#define AT_THREADS 320                             // loader, MMA issuer, and two softmax warps for each 32 rows
#define AT_WAIT_CYCLES 1000000000ll
#define AT_Q_BYTES (AT_QTILE * AT_HD * 2)
#define AT_STAGE_BYTES (2 * 2 * AT_KTILE * AT_HD * 2)   // keys, then values, of two pages and one head
#define AT_P_BYTES (AT_QTILE * 2 * AT_KTILE * 2)   // P of one step: the A operand of P.V, two panels of 64 keys
#define AT_TILE_BYTES (AT_Q_BYTES + AT_STAGES * AT_STAGE_BYTES + 2 * AT_P_BYTES)
#define AT_BAR_WORDS (13 + 2 * AT_STAGES)
#define AT_SMEM_BYTES (AT_TILE_BYTES + 8 * AT_BAR_WORDS + 8 * AT_STAGES + 2 * 2 * AT_QTILE * 4)
#define AT_TMEM_COLS 512                           // S buffers at columns 0 and 128, O from column 256
#define AT_O_COL 256
#define AT_LAZY 8.0f

struct AtArgs {
    bf16* out; const int* block_table; int table_stride; const int4* tiles;
    int nh, nkv, window; float scale_log2e;
    int pool_rows;                                 // rows of the key (and value) pool seen as a matrix [rows][head size]
};

__device__ __forceinline__ unsigned at_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool at_wait(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;                                          // the usual case costs neither a clock read nor a suspended wait
    const long long deadline = clock64() + AT_WAIT_CYCLES;
    for (;;) {
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() > deadline) return false;
    }
}
// the same for a whole warp: every lane gets the same answer, so the warp stays together on its way out
__device__ __forceinline__ bool at_wait_warp(unsigned bar, unsigned parity) {
    return __all_sync(0xffffffffu, at_wait(bar, parity));
}
__device__ __forceinline__ void at_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void at_tma_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// shared-memory operand descriptor, 128-byte swizzle: start address, leading and stride byte offsets
__device__ __forceinline__ unsigned long long at_desc(unsigned smem_addr, unsigned lbo, unsigned sbo) {
    return (unsigned long long)((smem_addr >> 4) & 0x3FFFu) | ((unsigned long long)((lbo >> 4) & 0x3FFFu) << 16) |
           ((unsigned long long)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void at_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void at_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 columns of this thread's lane.  at_ld32_start only issues the load: the values are there after at_ld_wait, and
// at_pin32 after that keeps the compiler from using the registers any earlier.
__device__ __forceinline__ void at_ld32_start(unsigned taddr, unsigned* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void at_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void at_pin32(unsigned* r) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                      "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                      "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                      "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}
__device__ __forceinline__ void at_ld32(unsigned taddr, float* v) {     // load and wait
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
__device__ __forceinline__ void at_st32(unsigned taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr),
                   "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
}
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// tiles[i] = (batch row, first packed token, number of tokens (<= AT_QTILE), position of the first token)
__global__ void __launch_bounds__(AT_THREADS, 1) attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                                  const __grid_constant__ CUtensorMap map_k,
                                                                                  const __grid_constant__ CUtensorMap map_v,
                                                                                  const AtArgs p, int* status) {
    // Q | stages of (K, V of two pages) | two P tiles | barriers and the stages' flags.  The tiles need 1024-byte
    // alignment for the swizzle, which the declaration asks for and the kernel checks.
    extern __shared__ __align__(1024) unsigned char at_mem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned q_s = at_smem(at_mem), kv_s = q_s + AT_Q_BYTES, p_s = kv_s + AT_STAGES * AT_STAGE_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(at_mem + AT_TILE_BYTES);
    unsigned long long &q_full = bars[0], &p_full = bars[1];
    unsigned long long *pv_done = bars + 2, *s_full = bars + 4, *s_free = bars + 6, *kv_full = bars + 8, *kv_empty = bars + 8 + AT_STAGES;
    unsigned long long* pair_bar = bars + 8 + 2 * AT_STAGES;       // one for the two softmax warps of each 32 rows
    unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(bars + 12 + 2 * AT_STAGES);
    volatile unsigned* stage_flags = reinterpret_cast<volatile unsigned*>(bars + AT_BAR_WORDS);   // bit g: page g of the stage exists
    float* exchange = reinterpret_cast<float*>(bars + AT_BAR_WORDS + AT_STAGES);    // [step parity][half][row]: what the halves of a row tell each other
    if (q_s & 1023u) {                                              // every thread alike: nothing is allocated yet
        if (threadIdx.x == 0) atomicExch(status, 6);
        return;
    }

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&q_full)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(at_smem(&p_full)) : "memory");          // the eight softmax warps
        for (int q = 0; q < 4; ++q) asm volatile("mbarrier.init.shared::cta.b64 [%0], 2;" ::"r"(at_smem(&pair_bar[q])) : "memory");
        for (int s = 0; s < AT_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&kv_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&kv_empty[s])) : "memory");
        }
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&s_full[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(at_smem(&s_free[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&pv_done[b])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(&tmem_base_s)), "r"((unsigned)AT_TMEM_COLS) : "memory");
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

    const int4 info = p.tiles[blockIdx.y];                          // heads vary fastest: the runs that see the most keys start first
    const int brow = info.x, tok0 = info.y, n = info.z, pos0 = info.w;
    const int h = blockIdx.x, kvh = h / (p.nh / p.nkv);
    // the pages the run can see: from the first row's window start to the last row's position, two to a step
    const int first_key = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int page_lo = first_key / AT_KTILE, page_hi = (pos0 + n - 1) / AT_KTILE;
    const int n_steps = (page_hi - page_lo + 2) / 2;

    if (warp == 0) {
        if (lane == 0) {                                            // ---------------- loader
            const int* table = p.block_table + (size_t)brow * p.table_stride;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(&q_full)), "r"((unsigned)AT_Q_BYTES) : "memory");
#pragma unroll
            for (int c = 0; c < AT_PANELS; ++c) at_tma_2d(q_s + c * (AT_QTILE * 128), &map_q, h * AT_HD + 64 * c, tok0, at_smem(&q_full));
            int page[2] = {table[page_lo], page_lo + 1 <= page_hi ? table[page_lo + 1] : -1};
            for (int it = 0; it < n_steps; ++it) {
                const int s = it % AT_STAGES;
                int next[2] = {-1, -1};                             // the step after this one: its entries travel during the wait
                if (page_lo + 2 * it + 2 <= page_hi) next[0] = table[page_lo + 2 * it + 2];
                if (page_lo + 2 * it + 3 <= page_hi) next[1] = table[page_lo + 2 * it + 3];
                if (it >= AT_STAGES && !at_wait(at_smem(&kv_empty[s]), (unsigned)((it / AT_STAGES) - 1) & 1u)) { atomicExch(status, 5); break; }
                const unsigned bar = at_smem(&kv_full[s]), k_dst = kv_s + s * AT_STAGE_BYTES, v_dst = k_dst + AT_STAGE_BYTES / 2;
                stage_flags[s] = (page[0] >= 0 ? 1u : 0u) | (page[1] >= 0 ? 2u : 0u);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((unsigned)AT_STAGE_BYTES) : "memory");
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    // a page that is not there (beyond the run's last page, or left behind by the window) is read from
                    // beyond the pool's end, which gives zeros: its scores are masked and its values add nothing
                    const int y = page[g] >= 0 ? (page[g] * p.nkv + kvh) * AT_KTILE : p.pool_rows;
#pragma unroll
                    for (int c = 0; c < AT_PANELS; ++c) {
                        at_tma_2d(k_dst + c * (2 * AT_KTILE * 128) + g * (AT_KTILE * 128), &map_k, 64 * c, y, bar);
                        at_tma_2d(v_dst + c * (2 * AT_KTILE * 128) + g * (AT_KTILE * 128), &map_v, 64 * c, y, bar);
                    }
                }
                page[0] = next[0]; page[1] = next[1];
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                            // ---------------- MMA issuer
            // instruction descriptors: float32 accumulator, bfloat16 operands, M = 128;
            // S: A and B K-major, N = 128 keys;  O: B MN-major (bit 16), N = head size
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)((2 * AT_KTILE) >> 3) << 17) | ((unsigned)(AT_QTILE >> 4) << 24);
            const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(AT_HD >> 3) << 17) | ((unsigned)(AT_QTILE >> 4) << 24);
            // operand descriptors of stage 0 and P tile 0; a stage or tile further on adds its offset in 16-byte units
            const unsigned long long dq = at_desc(q_s, 0, 1024), dk = at_desc(kv_s, 0, 1024), dp = at_desc(p_s, 0, 1024);
            const unsigned long long dv = at_desc(kv_s + AT_STAGE_BYTES / 2, 2 * AT_KTILE * 128, 1024);
            bool ok = at_wait(at_smem(&q_full), 0u);
            auto issue_s = [&](int it) -> bool {                    // S = Q . K^T of step `it` into S buffer it & 1
                const int s = it % AT_STAGES, b = it & 1;
                if (!at_wait(at_smem(&kv_full[s]), (unsigned)(it / AT_STAGES) & 1u)) return false;
                if (it >= 2 && !at_wait(at_smem(&s_free[b]), (unsigned)((it >> 1) - 1) & 1u)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long dks = dk + (unsigned long long)(s * (AT_STAGE_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < AT_HD / 16; ++kk) {           // 16 columns = 32 bytes inside the swizzle atom; 64 columns = one panel
                    const unsigned off_q = ((kk / 4) * (AT_QTILE * 128) + (kk % 4) * 32) >> 4, off_k = ((kk / 4) * (2 * AT_KTILE * 128) + (kk % 4) * 32) >> 4;
                    at_mma(tmem + b * (2 * AT_KTILE), dq + off_q, dks + off_k, idesc_s, kk > 0 ? 1u : 0u);
                }
                at_commit(at_smem(&s_full[b]));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int it = 0; it < n_steps && ok; ++it) {
                if (it + 1 < n_steps && !issue_s(it + 1)) { ok = false; break; }
                const int s = it % AT_STAGES, b = it & 1;
                if (!at_wait(at_smem(&p_full), (unsigned)it & 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long dps = dp + (unsigned long long)(b * (AT_P_BYTES >> 4)), dvs = dv + (unsigned long long)(s * (AT_STAGE_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < 2 * AT_KTILE / 16; ++kk) {    // 16 keys: 32 bytes further in P's rows (64 keys a panel), 16 rows further in V
                    const unsigned off_p = ((kk / 4) * (AT_QTILE * 128) + (kk % 4) * 32) >> 4, off_v = (kk * 16 * 128) >> 4;
                    at_mma(tmem + AT_O_COL, dps + off_p, dvs + off_v, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
                }
                at_commit(at_smem(&kv_empty[s]));                   // the stage's keys and values have been read
                at_commit(at_smem(&pv_done[b]));                    // and O holds this step's share
            }
            if (!ok) atomicExch(status, 5);
        }
    } else {                                                        // ---------------- softmax, warps 2..9
        // Two threads a query row: thread (row, g) has the scores of the step's page g (64 keys) and half of the
        // row of O.  The two tell each other their maxima, and at the end their sums, through shared memory.
        const int quarter = warp & 3;                               // the 32 lanes of tensor memory this warp may touch
        const int g = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;                          // this thread's query row
        const int p_r = pos0 + r;
        const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16);
        const unsigned o_addr = lane_addr + AT_O_COL + g * (AT_HD / 2);
        const unsigned pair = at_smem(&pair_bar[quarter]);
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        int it = 0, met = 0;                                        // met: how often the row's two threads have met
        // tell the other half `mine`, learn what it tells
        auto swap = [&](float mine, float& theirs) -> bool {
            float* slot = exchange + (met & 1) * (2 * AT_QTILE);
            slot[g * AT_QTILE + r] = mine;
            __syncwarp();
            if (lane == 0) at_arrive(pair);
            if (!at_wait_warp(pair, (unsigned)met & 1u)) return false;
            theirs = slot[(g ^ 1) * AT_QTILE + r];
            ++met;
            return true;
        };
        for (; it < n_steps; ++it) {
            const int b = it & 1, st = it % AT_STAGES;
            if (!at_wait_warp(at_smem(&kv_full[st]), (unsigned)(it / AT_STAGES) & 1u)) { ok = false; break; }   // the loader's flags
            const bool there = (stage_flags[st] >> g) & 1u;
            if (!at_wait_warp(at_smem(&s_full[b]), (unsigned)(it >> 1) & 1u)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int key0 = (page_lo + 2 * it + g) * AT_KTILE;
            unsigned raw[AT_KTILE];
            at_ld32_start(lane_addr + b * (2 * AT_KTILE) + g * AT_KTILE, raw);
            at_ld32_start(lane_addr + b * (2 * AT_KTILE) + g * AT_KTILE + 32, raw + 32);
            at_ld_wait();
            at_pin32(raw); at_pin32(raw + 32);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) at_arrive(at_smem(&s_free[b]));          // the buffer may take S of the step after next
            // the row sees the keys up to its own position and inside its window
            float s[AT_KTILE];
#pragma unroll
            for (int c = 0; c < AT_KTILE; ++c) s[c] = __uint_as_float(raw[c]);
            const bool whole = there && key0 + AT_KTILE - 1 <= p_r && (p.window <= 0 || key0 > p_r - p.window);
            if (!whole) {
#pragma unroll
                for (int c = 0; c < AT_KTILE; ++c) {
                    const int key = key0 + c;
                    if (!there || key > p_r || (p.window > 0 && key <= p_r - p.window)) s[c] = -INFINITY;
                }
            }
            float mx[4] = {s[0], s[1], s[2], s[3]};                 // four chains: a warp has little else to hide their latency
#pragma unroll
            for (int c = 4; c < AT_KTILE; ++c) mx[c & 3] = fmaxf(mx[c & 3], s[c]);
            const float m_mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            float m_theirs;
            if (!swap(m_mine, m_theirs)) { ok = false; break; }
            // The reference point of the exponentials follows the row's maximum only when that has grown by more than
            // AT_LAZY (in powers of two): P then holds values up to 2^AT_LAZY, which bfloat16 and the float32 sums take
            // as well as values up to 1, and O is rescaled on few steps instead of on nearly all.  Both threads of a
            // row compute the same from the same numbers.
            const float m_tile = fmaxf(m_mine, m_theirs) * p.scale_log2e;
            const float m_new = (m_run != -INFINITY && m_tile <= m_run + AT_LAZY) ? m_run : fmaxf(m_run, m_tile);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = m_run == -INFINITY ? 1.0f : at_exp2(m_run - m_use);
            m_run = m_new;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            unsigned packed[AT_KTILE / 2];
#pragma unroll
            for (int c = 0; c < AT_KTILE; c += 2) {
                const float e0 = at_exp2(fmaf(s[c], p.scale_log2e, -m_use)), e1 = at_exp2(fmaf(s[c + 1], p.scale_log2e, -m_use));
                sum[c & 3] += e0; sum[(c + 1) & 3] += e1;
                packed[c >> 1] = at_pack(e0, e1);
            }
            l_run = l_run * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
            // this P tile is free once P.V of the step before last is done
            if (it >= 2 && !at_wait_warp(at_smem(&pv_done[b]), (unsigned)((it >> 1) - 1) & 1u)) { ok = false; break; }
            if (it > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) { // a row's reference point moved: rescale this half of the warp's rows of O
                if (!at_wait_warp(at_smem(&pv_done[b ^ 1]), (unsigned)((it - 1) >> 1) & 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c = 0; c < AT_HD / 2; c += 32) {
                    float o[32];
                    at_ld32(o_addr + c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= alpha;
                    at_st32(o_addr + c, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // P as bfloat16 for P.V: panel g of the tile (64 keys = 128 bytes a row)
            unsigned char* p_row = at_mem + (p_s - q_s) + b * AT_P_BYTES + g * (AT_QTILE * 128) + r * 128;
#pragma unroll
            for (int c = 0; c < AT_KTILE / 8; ++c)
                *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core's proxy
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) at_arrive(at_smem(&p_full));
        }
        // the row's sum, and the last P.V (products complete in the order they were issued)
        float l_theirs = 0.f;
        if (ok && !swap(l_run, l_theirs)) ok = false;
        if (ok && it > 0 && !at_wait_warp(at_smem(&pv_done[(it - 1) & 1]), (unsigned)((it - 1) >> 1) & 1u)) ok = false;
        if (ok && it > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float l = g == 0 ? l_run + l_theirs : l_theirs + l_run;   // the same sum in both threads
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* o_row = p.out + ((size_t)(tok0 + r) * p.nh + h) * AT_HD + g * (AT_HD / 2);
#pragma unroll 1
            for (int c = 0; c < AT_HD / 2; c += 32) {
                float o[32];
                at_ld32(o_addr + c, o);
                if (r < n) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(o_row + c + i) = make_uint4(at_pack(o[i] * inv, o[i + 1] * inv), at_pack(o[i + 2] * inv, o[i + 3] * inv),
                                                                              at_pack(o[i + 4] * inv, o[i + 5] * inv), at_pack(o[i + 6] * inv, o[i + 7] * inv));
                }
            }
        }
        if (!ok) atomicExch(status, 5);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)AT_TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
namespace {

typedef CUresult (*at_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

at_encode_fn at_encoder() {
    static at_encode_fn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (at_encode_fn)sym;
    }
    return fn;
}

// a bfloat16 matrix of `rows` rows of `cols` columns, `stride` elements apart, read in boxes of 64 columns x box_rows rows
int at_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long stride, int box_rows) {
    at_encode_fn enc = at_encoder();
    if (!enc) return PE_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace

extern "C" int pe_attention_prefill_tcgen05_tile() { return AT_QTILE; }

// how many of the kernel's CTAs an SM holds at once (one: it takes all of tensor memory), or a negative CUDA error
extern "C" int pe_attention_prefill_tcgen05_ctas_per_sm() {
    int n = 0;
    if (cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM_BYTES) != cudaSuccess) return -1;
    const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_prefill_tcgen05_kernel, AT_THREADS, AT_SMEM_BYTES);
    return e == cudaSuccess ? n : -(int)e;
}

// q: [n_tokens][q_stride] with head h at columns h * hd; pools: [pool_pages][nkv][64][hd]
extern "C" int pe_attention_prefill_tcgen05(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                            long long pool_pages, const int* block_table, int table_stride, const void* tiles,
                                            int n_tiles, int n_tokens, int nh, int nkv, int hd, int window, float scale,
                                            int* status, void* stream) {
    if (n_tiles <= 0) return 0;
    if (hd != AT_HD || nkv <= 0 || nh % nkv || n_tiles > 65535 || q_stride % 8 || !(scale > 0.f) || !status) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out | (uintptr_t)tiles) & 15) return PE_ERR_UNSUPPORTED;
    if (pool_pages * nkv * AT_KTILE > 0x7fffff00ll) return PE_ERR_UNSUPPORTED;       // TMA coordinates are 32-bit
    CUtensorMap mq, mk, mv;
    int rc = at_make_map(&mq, q, n_tokens, (long long)nh * hd, q_stride, AT_QTILE);
    if (rc) return rc;
    rc = at_make_map(&mk, k_pool, pool_pages * nkv * AT_KTILE, hd, hd, AT_KTILE);
    if (rc) return rc;
    rc = at_make_map(&mv, v_pool, pool_pages * nkv * AT_KTILE, hd, hd, AT_KTILE);
    if (rc) return rc;
    AtArgs p = {};
    p.out = (bf16*)out; p.block_table = block_table; p.table_stride = table_stride; p.tiles = (const int4*)tiles;
    p.nh = nh; p.nkv = nkv; p.window = window; p.scale_log2e = scale * 1.4426950408889634f;
    p.pool_rows = (int)(pool_pages * nkv * AT_KTILE);
    const size_t smem = AT_SMEM_BYTES;
    static bool attr_set = false;
    if (!attr_set) {
        PE_TRY(cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    PE_TRY(pe_launch(attention_prefill_tcgen05_kernel, dim3(nh, n_tiles), AT_THREADS, smem, (cudaStream_t)stream, mq, mk, mv, p, status));
    return 0;
}

#else   // other head sizes: the mma.sync kernel of attention_prefill.cu takes them

extern "C" int pe_attention_prefill_tcgen05_tile() { return 0; }
extern "C" int pe_attention_prefill_tcgen05_ctas_per_sm() { return 0; }
extern "C" int pe_attention_prefill_tcgen05(const void*, int, void*, const void*, const void*, long long, const int*, int, const void*,
                                            int, int, int, int, int, int, float, int*, void*) {
    return PE_ERR_UNSUPPORTED;
}

#endif
