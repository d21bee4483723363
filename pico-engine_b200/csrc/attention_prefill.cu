// Causal attention of many tokens per sequence over the paged bfloat16 cache (prompts, or any
// step that brings more than one token per sequence), compiled for one head size
// (PE_HEAD_DIM).  Keys and values are read from the cache pages, which already hold this
// step's tokens, so a sequence may continue from any earlier length.
//
// Flash-attention tiling.  Grid: (run of up to 64 consecutive tokens of one sequence, query
// head); eight warps: two for each 16 query rows, which take the even and the odd pages of the
// run's keys and merge their results at the end (the CTAs of a prompt are resident together, so
// the kernel lasts as long as the run that sees the most keys; two warps shorten that run, which
// gains 5 % at 4,096 tokens and little at 2,048, where the SMs' issue rate is the limit).  A page of
// the cache (64 keys of one kv head) is one contiguous tile: the CTA brings pairs of key and
// value pages into shared memory with cp.async, three stages deep, XOR-swizzled in 16-byte
// chunks so that ldmatrix reads are free of bank conflicts; S = Q.K^T and O += P.V run on
// mma.sync m16n8k16 with fragments from ldmatrix (values through ldmatrix.trans); softmax
// statistics are float32 per row in registers.  Pages that lie wholly outside what a warp's
// rows may see (beyond the diagonal, or before the window) are skipped by that warp.
//
// pico-engine hands this to torch's fused attention after copying keys and values out of the
// cache (src/pico_engine/model.py:201-209).
#ifndef PE_HEAD_DIM
#error "compile with -DPE_HEAD_DIM=<head size>"
#endif
#include "common.cuh"

#define AP_HD PE_HEAD_DIM
#define AP_ROW_WARPS 4                             // 64 query rows a CTA: several CTAs share an SM and hide each other's waits
#define AP_SPLIT (AP_HD <= 128 ? 2 : 1)            // warps a row group (larger heads: no room for pairs of pages)
#define AP_WARPS (AP_SPLIT * AP_ROW_WARPS)         // two warps a row group: even and odd pages
#define AP_QTILE (16 * AP_ROW_WARPS)
#define AP_KTILE PE_PAGE
#define AP_STAGES 3                                // key/value pages in flight or in use
#define AP_CHUNKS (AP_HD / 8)                      // 16-byte chunks in a row
#define AP_SWIZZLE ((AP_CHUNKS % 8) == 0)          // rows of a multiple of 128 bytes: XOR the chunk with the row
#define AP_NT (AP_HD / 8)                          // 8-wide output tiles
#define AP_KS (AP_HD / 16)                         // 16-deep steps over the head dimension

__device__ __forceinline__ unsigned ap_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned ap_offset(int row, int chunk) {   // byte offset of a 16-byte chunk in a tile
    return (unsigned)(row * AP_HD * 2 + ((AP_SWIZZLE ? (chunk ^ (row & 7)) : chunk) << 4));
}
__device__ __forceinline__ void ap_cp16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ap_ldmatrix(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ap_ldmatrix_t(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ap_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (relative error about 2^-22): the softmax of a tile needs 16 of
// them per lane and row, and the exact routine would cost as much as the tile's MMAs
__device__ __forceinline__ float ap_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned ap_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// tiles[i] = (batch row, first packed token, number of tokens (<= AP_QTILE), position of the first token)
__global__ void __launch_bounds__(32 * AP_WARPS, AP_HD <= 64 ? 2 : 1) attention_prefill_kernel(
    const bf16* q, int q_stride, bf16* out, const bf16* k_pool, const bf16* v_pool, const int* block_table,
    int table_stride, const int4* tiles, int nh, int nkv, int window, float scale_log2e) {
    extern __shared__ __align__(128) unsigned char ap_mem[];     // Q [64][HD], then K and V [AP_STAGES][2 pages][64][HD] each
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & (AP_ROW_WARPS - 1), half = tid / (32 * AP_ROW_WARPS), g = lane >> 2, t = lane & 3;
    const int4 info = tiles[blockIdx.x];
    const int brow = info.x, tok0 = info.y, n = info.z, pos0 = info.w;
    const int h = blockIdx.y, kvh = h / (nh / nkv);
    const int* table = block_table + (size_t)brow * table_stride;

    const unsigned q_s = ap_smem(ap_mem);
    const unsigned tile_bytes = AP_KTILE * AP_HD * 2;
    const unsigned k_s = q_s + AP_QTILE * AP_HD * 2, v_s = k_s + AP_SPLIT * AP_STAGES * tile_bytes;

    // the pages the run can see: from the first row's window start to the last row's position
    const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int page_lo = first_key / AP_KTILE, page_hi = (pos0 + n - 1) / AP_KTILE;

    // pair `pr` of pages (page_lo + 2 pr and the next) into a stage; all threads; bit h of the result: page h is there
    auto load_pair = [&](int pr, int stage) -> int {
        int there = 0;
#pragma unroll
        for (int h2 = 0; h2 < AP_SPLIT; ++h2) {
            const int pi = page_lo + AP_SPLIT * pr + h2;
            if (pi > page_hi) continue;
            const int page = table[pi];
            if (page < 0) continue;                              // a page the window has left behind
            there |= 1 << h2;
            const size_t base = ((size_t)page * nkv + kvh) * AP_KTILE * AP_HD;
            for (int idx = tid; idx < AP_KTILE * AP_CHUNKS; idx += 32 * AP_WARPS) {
                const int row = idx / AP_CHUNKS, chunk = idx % AP_CHUNKS;
                const unsigned off = (AP_SPLIT * stage + h2) * tile_bytes + ap_offset(row, chunk);
                ap_cp16(k_s + off, k_pool + base + (size_t)row * AP_HD + chunk * 8);
                ap_cp16(v_s + off, v_pool + base + (size_t)row * AP_HD + chunk * 8);
            }
        }
        return there;
    };

    // Q rows of the run (zeros beyond its end)
    for (int idx = tid; idx < AP_QTILE * AP_CHUNKS; idx += 32 * AP_WARPS) {
        const int row = idx / AP_CHUNKS, chunk = idx % AP_CHUNKS;
        if (row < n) ap_cp16(q_s + ap_offset(row, chunk), q + (size_t)(tok0 + row) * q_stride + (size_t)h * AP_HD + chunk * 8);
        else *reinterpret_cast<uint4*>(ap_mem + ap_offset(row, chunk)) = make_uint4(0u, 0u, 0u, 0u);
    }
    // the first AP_STAGES - 1 pairs of pages are requested at once, one commit group each (empty groups keep the count)
    const int n_pairs = (page_hi - page_lo + AP_SPLIT) / AP_SPLIT;
    int pair_ok[AP_STAGES];
#pragma unroll
    for (int i = 0; i < AP_STAGES - 1; ++i) {
        pair_ok[i] = i < n_pairs ? load_pair(i, i) : 0;
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // this warp's rows
    const int i_lo = warp * 16 + g, i_hi = i_lo + 8;
    const bool row_lo = i_lo < n, row_hi = i_hi < n;
    const int p_lo = pos0 + i_lo, p_hi = pos0 + i_hi;
    const int w_first = pos0 + warp * 16, w_last = pos0 + min(n, warp * 16 + 16) - 1;   // positions of the warp's rows
    const bool warp_has_rows = warp * 16 < n;

    unsigned qf[AP_KS][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[AP_NT][4];
#pragma unroll
    for (int j = 0; j < AP_NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

    const int mat = lane >> 3, mr = lane & 7;
    for (int it = 0; it < n_pairs; ++it) {
        const int stage = it % AP_STAGES, ahead = (it + AP_STAGES - 1) % AP_STAGES;
        const int pi = page_lo + AP_SPLIT * it + half;            // this warp's page of the pair
        asm volatile("cp.async.wait_group %0;" ::"n"(AP_STAGES - 2) : "memory");   // this iteration's pages (and Q) have landed
        __syncthreads();                                          // ... for every thread; and all warps are done with the last pair
        // the pair AP_STAGES - 1 ahead goes into the stage that the previous iteration used
        pair_ok[ahead] = it + AP_STAGES - 1 < n_pairs ? load_pair(it + AP_STAGES - 1, ahead) : 0;
        asm volatile("cp.async.commit_group;" ::: "memory");
        const bool ok_cur = (pair_ok[stage] >> half) & 1;
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < AP_KS; ++ks)
                ap_ldmatrix(qf[ks], q_s + ap_offset(warp * 16 + mr + (mat & 1) * 8, 2 * ks + (mat >> 1)));
        }
        const int key0 = pi * AP_KTILE;
        const bool visible = ok_cur && warp_has_rows && key0 <= w_last &&
                             (window <= 0 || key0 + AP_KTILE - 1 >= w_first - window + 1);
        if (visible) {
            const unsigned kt = k_s + (AP_SPLIT * stage + half) * tile_bytes, vt = v_s + (AP_SPLIT * stage + half) * tile_bytes;
            float s[AP_KTILE / 8][4];
#pragma unroll
            for (int j = 0; j < AP_KTILE / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < AP_KS; ++ks)
#pragma unroll
                for (int jj = 0; jj < AP_KTILE / 16; ++jj) {     // 16 keys: two 8-key tiles
                    unsigned b[4];
                    ap_ldmatrix(b, kt + ap_offset(jj * 16 + mr + (mat >> 1) * 8, 2 * ks + (mat & 1)));
                    ap_mma(s[2 * jj], qf[ks], b[0], b[1]);
                    ap_mma(s[2 * jj + 1], qf[ks], b[2], b[3]);
                }
            // scale, mask, running maximum.  s[j][e]: row (e & 2 ? g + 8 : g), key key0 + j*8 + 2t + (e & 1)
            // A page that every row of the warp sees whole (before the diagonal, inside the window) needs no mask.
            const bool whole = key0 + AP_KTILE - 1 <= w_first && w_last < pos0 + n && warp * 16 + 16 <= n &&
                               (window <= 0 || w_last - key0 < window);
            float tmax[2] = {-INFINITY, -INFINITY};
            if (whole) {
#pragma unroll
                for (int j = 0; j < AP_KTILE / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) tmax[e >> 1] = fmaxf(tmax[e >> 1], s[j][e]);
                tmax[0] *= scale_log2e; tmax[1] *= scale_log2e;
            } else {
#pragma unroll
                for (int j = 0; j < AP_KTILE / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + 2 * t + (e & 1);
                        const int p = (e & 2) ? p_hi : p_lo;
                        const bool see = ((e & 2) ? row_hi : row_lo) && key <= p && (window <= 0 || p - key < window);
                        if (!see) s[j][e] = -INFINITY;
                        tmax[e >> 1] = fmaxf(tmax[e >> 1], s[j][e] * scale_log2e);
                    }
            }
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
                const float m_new = fmaxf(m_run[r], tmax[r]);
                alpha[r] = (m_run[r] == -INFINITY) ? 0.f : ap_exp2(m_run[r] - m_new);
                m_run[r] = m_new;
                l_run[r] *= alpha[r];
            }
            // a row that has seen no key yet has the maximum -inf: its exponents are taken against 0, and are all 0
            const float m_use[2] = {m_run[0] == -INFINITY ? 0.f : m_run[0], m_run[1] == -INFINITY ? 0.f : m_run[1]};
#pragma unroll
            for (int j = 0; j < AP_KTILE / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = ap_exp2(fmaf(s[j][e], scale_log2e, -m_use[e >> 1]));      // 2^-inf = 0
                    s[j][e] = pv;
                    l_run[e >> 1] += pv;
                }
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {                 // seldom after the first pages
#pragma unroll
                for (int j = 0; j < AP_NT; ++j) {
                    o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < AP_KTILE / 16; ++kk) {         // 16 keys at a time
                unsigned pa[4];
                pa[0] = ap_pack(s[2 * kk][0], s[2 * kk][1]);         pa[1] = ap_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = ap_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]); pa[3] = ap_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int nt = 0; nt < AP_NT; nt += 2) {          // two 8-wide tiles of the head dimension
                    unsigned b[4];
                    ap_ldmatrix_t(b, vt + ap_offset(kk * 16 + mr + (mat & 1) * 8, nt + (mat >> 1)));
                    ap_mma(o[nt], pa, b[0], b[1]);
                    ap_mma(o[nt + 1], pa, b[2], b[3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    // the warps of the odd pages hand their (max, sum, O) to their partners through shared memory (the stages are free)
    if (AP_SPLIT == 2) {
    __syncthreads();
    float* hand = reinterpret_cast<float*>(ap_mem + AP_QTILE * AP_HD * 2) + (size_t)(tid % (32 * AP_ROW_WARPS)) * (4 * AP_NT + 4);
    if (half == 1) {
#pragma unroll
        for (int j = 0; j < AP_NT; ++j) *reinterpret_cast<float4*>(hand + 4 * j) = make_float4(o[j][0], o[j][1], o[j][2], o[j][3]);
        *reinterpret_cast<float4*>(hand + 4 * AP_NT) = make_float4(m_run[0], m_run[1], l_run[0], l_run[1]);
    }
    __syncthreads();
    if (half == 1) return;
    {
        const float4 ml = *reinterpret_cast<const float4*>(hand + 4 * AP_NT);
        const float m_other[2] = {ml.x, ml.y}, l_other[2] = {ml.z, ml.w};
        float mine_s[2], other_s[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float m = fmaxf(m_run[r], m_other[r]);
            mine_s[r] = m_run[r] == -INFINITY ? 0.f : ap_exp2(m_run[r] - m);
            other_s[r] = m_other[r] == -INFINITY ? 0.f : ap_exp2(m_other[r] - m);
            l_run[r] = l_run[r] * mine_s[r] + l_other[r] * other_s[r];
        }
#pragma unroll
        for (int j = 0; j < AP_NT; ++j) {
            const float4 x = *reinterpret_cast<const float4*>(hand + 4 * j);
            o[j][0] = o[j][0] * mine_s[0] + x.x * other_s[0]; o[j][1] = o[j][1] * mine_s[0] + x.y * other_s[0];
            o[j][2] = o[j][2] * mine_s[1] + x.z * other_s[1]; o[j][3] = o[j][3] * mine_s[1] + x.w * other_s[1];
        }
    }
    }
    const float inv_lo = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv_hi = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
#pragma unroll
    for (int j = 0; j < AP_NT; ++j) {
        const int col = j * 8 + 2 * t;
        if (row_lo)
            *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + i_lo) * nh + h) * AP_HD + col) = ap_pack(o[j][0] * inv_lo, o[j][1] * inv_lo);
        if (row_hi)
            *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + i_hi) * nh + h) * AP_HD + col) = ap_pack(o[j][2] * inv_hi, o[j][3] * inv_hi);
    }
}

extern "C" int pe_attention_prefill_tile() { return AP_QTILE; }

extern "C" int pe_attention_prefill(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                    const int* block_table, int table_stride, const void* tiles, const int* unused0,
                                    const int* unused1, int n_tiles, int nh, int nkv, int hd, int window, float scale,
                                    void* stream) {
    (void)unused0; (void)unused1;
    if (n_tiles <= 0) return 0;
    if (hd != AP_HD || nkv <= 0 || nh % nkv || nh > 65535 || q_stride % 8) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out | (uintptr_t)tiles) & 15) return PE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(AP_QTILE + 2 * AP_SPLIT * AP_STAGES * AP_KTILE) * AP_HD * 2;   // Q, then K and V pages
    static bool attr_set = false;
    if (smem > 48 * 1024 && !attr_set) {
        PE_TRY(cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    dim3 grid(n_tiles, nh);
    PE_TRY(pe_launch(attention_prefill_kernel, grid, 32 * AP_WARPS, smem, (cudaStream_t)stream,
                     (const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_stride,
                     (const int4*)tiles, nh, nkv, window, scale * 1.4426950408889634f));
    return 0;
}
