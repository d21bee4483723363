// Causal attention of many tokens per sequence over the paged bfloat16 cache (prompts, or any
// step that brings more than one token per sequence), compiled for one head size
// (PE_HEAD_DIM).  Keys and values are read from the cache pages, which already hold this
// step's tokens, so a sequence may continue from any earlier length.
//
// Grid: (tile of up to 64 consecutive tokens of one sequence, query head).  Each of the four
// warps owns 16 query rows and walks the keys its rows can see in tiles of 16, with the next
// tile's loads in flight while the current one is in the tensor cores (mma.sync m16n8k16;
// the fragment scheme is that of attention_mma.cuh).  Warps do not synchronise.
//
// pico-engine hands this to torch's fused attention after copying keys and values out of the
// cache (src/pico_engine/model.py:201-209).
#ifndef PE_HEAD_DIM
#error "compile with -DPE_HEAD_DIM=<head size>"
#endif
#include "attention_mma.cuh"

#define AP_WARPS 4
#define AP_QTILE (16 * AP_WARPS)

// tiles[i] = (batch row, first packed token, number of tokens (<= AP_QTILE), position of the first token)
__global__ void __launch_bounds__(32 * AP_WARPS) attention_prefill_kernel(
    const bf16* q, int q_stride, bf16* out, const bf16* k_pool,
    const bf16* v_pool, const int* block_table, int table_stride,
    const int4* tiles, int nh, int nkv, int window, float scale_log2e) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int4 info = tiles[blockIdx.x];
    const int brow = info.x, tok0 = info.y, n = info.z, pos0 = info.w;
    const int h = blockIdx.y, kvh = h / (nh / nkv);
    if (warp * 16 >= n) return;
    const int* table = block_table + (size_t)brow * table_stride;
    const int i_lo = warp * 16 + g, i_hi = i_lo + 8;             // this lane's two query rows within the tile
    const bool ok_lo = i_lo < n, ok_hi = i_hi < n;
    const int p_lo = pos0 + i_lo, p_hi = pos0 + i_hi;            // their positions
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 qf[AM_NCHUNK][2];
#pragma unroll
    for (int c = 0; c < AM_NCHUNK; ++c) {
        const int col = c * 32 + t * 8;
        const bool cin = col + 8 <= AM_HD;
        const bf16* qp = q + (size_t)h * AM_HD + col;
        qf[c][0] = (cin && ok_lo) ? am_ld16(qp + (size_t)(tok0 + i_lo) * q_stride) : zero;
        qf[c][1] = (cin && ok_hi) ? am_ld16(qp + (size_t)(tok0 + i_hi) * q_stride) : zero;
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[AM_NCHUNK][4][4];
#pragma unroll
    for (int c = 0; c < AM_NCHUNK; ++c)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[c][r][0] = acc[c][r][1] = acc[c][r][2] = acc[c][r][3] = 0.f;

    // keys this warp's rows can see: from the first row's window start to the last row's position
    const int w_first = pos0 + warp * 16, w_last = pos0 + min(n, warp * 16 + 16) - 1;
    const int k_lo = (window > 0 && w_first - window + 1 > 0) ? w_first - window + 1 : 0;
    const int tile_end = w_last / 16;                            // inclusive
    int tile = k_lo / 16;

    // software pipeline: `next` is loaded while `cur` is used
    AmTile cur, next;
    bool cur_ok = false, next_ok = false;
    int cur_key0 = 0;
    auto fetch = [&](AmTile& dst, int tl, bool& ok) {
        ok = false;
        if (tl > tile_end) return;
        const int key0 = tl * 16;
        const int page = table[key0 / PE_PAGE];
        if (page < 0) return;                                    // left behind by the window
        am_load_tile(dst, k_pool, v_pool, (((size_t)page * nkv + kvh) * PE_PAGE + (key0 % PE_PAGE)) * AM_HD, g, t);
        ok = true;
    };
    fetch(cur, tile, cur_ok);
    cur_key0 = tile * 16;
    for (; tile <= tile_end; ++tile) {
        fetch(next, tile + 1, next_ok);
        if (cur_ok) {
            float s[2][4];
            am_scores(s, qf, cur);
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = cur_key0 + j * 8 + 2 * t + (e & 1);
                    const int p = (e & 2) ? p_hi : p_lo;
                    const bool ok = ((e & 2) ? ok_hi : ok_lo) && key <= p && (window <= 0 || p - key < window);
                    s[j][e] = ok ? s[j][e] * scale_log2e : -INFINITY;
                }
            am_softmax_accumulate(s, m_run, l_run, acc, cur);
        }
        cur = next;
        cur_ok = next_ok;
        cur_key0 = (tile + 1) * 16;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv_lo = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv_hi = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
#pragma unroll
    for (int c = 0; c < AM_NCHUNK; ++c) {
        const int col = c * 32 + t * 8;                          // this lane's 8 consecutive columns of the chunk
        if (col + 8 > AM_HD) continue;
        if (ok_lo) {
            uint4 v;
            v.x = am_pack(acc[c][0][0] * inv_lo, acc[c][0][1] * inv_lo); v.y = am_pack(acc[c][1][0] * inv_lo, acc[c][1][1] * inv_lo);
            v.z = am_pack(acc[c][2][0] * inv_lo, acc[c][2][1] * inv_lo); v.w = am_pack(acc[c][3][0] * inv_lo, acc[c][3][1] * inv_lo);
            *reinterpret_cast<uint4*>(out + ((size_t)(tok0 + i_lo) * nh + h) * AM_HD + col) = v;
        }
        if (ok_hi) {
            uint4 v;
            v.x = am_pack(acc[c][0][2] * inv_hi, acc[c][0][3] * inv_hi); v.y = am_pack(acc[c][1][2] * inv_hi, acc[c][1][3] * inv_hi);
            v.z = am_pack(acc[c][2][2] * inv_hi, acc[c][2][3] * inv_hi); v.w = am_pack(acc[c][3][2] * inv_hi, acc[c][3][3] * inv_hi);
            *reinterpret_cast<uint4*>(out + ((size_t)(tok0 + i_hi) * nh + h) * AM_HD + col) = v;
        }
    }
}

extern "C" int pe_attention_prefill(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                    const int* block_table, int table_stride, const void* tiles, const int* unused0,
                                    const int* unused1, int n_tiles, int nh, int nkv, int hd, int window, float scale,
                                    void* stream) {
    (void)unused0; (void)unused1;
    if (n_tiles <= 0) return 0;
    if (hd != AM_HD || nkv <= 0 || nh % nkv || nh > 65535 || q_stride % 8) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out | (uintptr_t)tiles) & 15) return PE_ERR_UNSUPPORTED;
    dim3 grid(n_tiles, nh);
    PE_TRY(pe_launch(attention_prefill_kernel, grid, 32 * AP_WARPS, 0, (cudaStream_t)stream, 
        (const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_stride,
        (const int4*)tiles, nh, nkv, window, scale * 1.4426950408889634f));
    PE_LAUNCH_CHECK();
    return 0;
}
