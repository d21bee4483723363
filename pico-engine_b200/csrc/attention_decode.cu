// Attention of single tokens over the paged bfloat16 cache (decoding), compiled for one head
// size (PE_HEAD_DIM, a multiple of 16 up to 256).
//
// Grid: (token, kv head x tile of 16 query heads, range of keys).  All query heads that share
// a kv head sit in the 16 rows of one MMA tile, so keys and values are read once for the
// group.  A warp takes 16 keys at a time: scores S = Q.K^T with mma.sync m16n8k16 (keys are
// loaded from global memory straight into B fragments with 16-byte loads, the head dimension
// permuted identically in Q), online softmax in float32 on the accumulator registers, then
// O += P.V where V fragments come from 16-byte row loads transposed in registers with
// movmatrix.  No shared memory until the four warps of a CTA merge their (max, sum, O).
// Key ranges are merged by a second small kernel from float32 partials in scratch.
//
// pico-engine's counterpart is _decode_attn_fwd (src/pico_engine/kernels.py:90-126): one
// program per query head, looping over the whole buffer.
#ifndef PE_HEAD_DIM
#error "compile with -DPE_HEAD_DIM=<head size>"
#endif
#include "attention_mma.cuh"

#define AD_WARPS 4
#define AD_HD PE_HEAD_DIM
#define AD_NCHUNK ((AD_HD + 31) / 32)
#define AD_ROW (AD_HD + 2)                 // floats per merged row in shared memory: O, max, sum

__global__ void __launch_bounds__(32 * AD_WARPS) attention_decode_kernel(
    const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool,
    const int* block_table, int table_stride, const int* tok_pos,
    const int* tok_row, int nh, int nkv, int window, float scale_log2e, int split_len, int n_splits,
    float* part, bf16* out) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];                       // [AD_WARPS][16][AD_ROW]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int tok = blockIdx.x, split = blockIdx.z;
    const int G = nh / nkv, head_tiles = (G + 15) / 16;
    const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y % head_tiles;
    const int pos = tok_pos[tok];
    const int* table = block_table + (size_t)tok_row[tok] * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int r_lo = ht * 16 + g, r_hi = r_lo + 8;        // this lane's two query heads within the group
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 qf[AD_NCHUNK][2];
#pragma unroll
    for (int c = 0; c < AD_NCHUNK; ++c) {
        const int col = c * 32 + t * 8;
        const bool cin = col + 8 <= AD_HD;
        const bf16* qp = q + (size_t)tok * q_stride + col;
        qf[c][0] = (cin && r_lo < G) ? am_ld16(qp + (size_t)(kvh * G + r_lo) * AD_HD) : zero;
        qf[c][1] = (cin && r_hi < G) ? am_ld16(qp + (size_t)(kvh * G + r_hi) * AD_HD) : zero;
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[AD_NCHUNK][4][4];
#pragma unroll
    for (int c = 0; c < AD_NCHUNK; ++c)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[c][r][0] = acc[c][r][1] = acc[c][r][2] = acc[c][r][3] = 0.f;

    const int begin = max(lo, split * split_len), end = min(pos + 1, (split + 1) * split_len);
    // software pipeline: the loads of the warp's next tile are in flight while the current one is used
    AmTile cur, next;
    bool cur_ok = false, next_ok = false;
    auto fetch = [&](AmTile& dst, int tl, bool& ok) {
        ok = false;
        if (tl * 16 >= end) return;
        const int page = table[tl * 16 / PE_PAGE];
        if (page < 0) return;                             // a page the window has left behind
        am_load_tile(dst, k_pool, v_pool, (((size_t)page * nkv + kvh) * PE_PAGE + (tl * 16 % PE_PAGE)) * AD_HD, g, t);
        ok = true;
    };
    int tile = begin / 16 + warp;
    fetch(cur, tile, cur_ok);
    for (; tile * 16 < end; tile += AD_WARPS) {
        fetch(next, tile + AD_WARPS, next_ok);
        if (cur_ok) {
            const int key0 = tile * 16;
            float s[2][4];
            am_scores(s, qf, cur);
            // s[j][e]: row (e & 2 ? g + 8 : g), key key0 + j*8 + 2t + (e & 1)
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + 2 * t + (e & 1);
                    s[j][e] = (key >= begin && key < end) ? s[j][e] * scale_log2e : -INFINITY;
                }
            am_softmax_accumulate(s, m_run, l_run, acc, cur);
        }
        cur = next;
        cur_ok = next_ok;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }

    // merge the warps: smem[warp][row][0..HD) = O, [HD] = max, [HD+1] = sum
    float* mine = smem + (size_t)warp * 16 * AD_ROW;
#pragma unroll
    for (int c = 0; c < AD_NCHUNK; ++c)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int col = c * 32 + t * 8 + 2 * r;       // acc[c][r][0..1]: row g, cols col, col+1; [2..3]: row g+8
            if (col < AD_HD) {
                mine[g * AD_ROW + col] = acc[c][r][0];       mine[g * AD_ROW + col + 1] = acc[c][r][1];
                mine[(g + 8) * AD_ROW + col] = acc[c][r][2]; mine[(g + 8) * AD_ROW + col + 1] = acc[c][r][3];
            }
        }
    if (t == 0) {
        mine[g * AD_ROW + AD_HD] = m_run[0];       mine[g * AD_ROW + AD_HD + 1] = l_run[0];
        mine[(g + 8) * AD_ROW + AD_HD] = m_run[1]; mine[(g + 8) * AD_ROW + AD_HD + 1] = l_run[1];
    }
    __syncthreads();
    const int rows = min(16, G - ht * 16);
    for (int idx = threadIdx.x; idx < rows * AD_HD; idx += blockDim.x) {
        const int row = idx / AD_HD, col = idx % AD_HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) m = fmaxf(m, smem[((size_t)w * 16 + row) * AD_ROW + AD_HD]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float* src = smem + ((size_t)w * 16 + row) * AD_ROW;
            const float wgt = (src[AD_HD] == -INFINITY) ? 0.f : exp2f(src[AD_HD] - m);
            o = fmaf(src[col], wgt, o);
            l = fmaf(src[AD_HD + 1], wgt, l);
        }
        const int head = kvh * G + ht * 16 + row;
        if (n_splits == 1) {
            out[((size_t)tok * nh + head) * AD_HD + col] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            float* dst = part + (((size_t)tok * nh + head) * n_splits + split) * AD_ROW;
            dst[col] = o;
            if (col == 0) { dst[AD_HD] = m; dst[AD_HD + 1] = l; }
        }
    }
}

// out[token][head][:] from the partials of all key ranges.  One block per (token, head); its
// threads are AD_MERGE_GROUPS groups that each take every AD_MERGE_GROUPS-th range (so that the
// loads of many ranges are in flight at once) and then add their sums in the order of the groups.
#define AD_MERGE_GROUPS 4
#define AD_MERGE_COLS (AD_HD < 32 ? 32 : AD_HD)

__global__ void __launch_bounds__(AD_MERGE_GROUPS * AD_MERGE_COLS) attention_decode_merge_kernel(
    const float* part, int n_splits, bf16* out) {
    __shared__ float o_s[AD_MERGE_GROUPS][AD_MERGE_COLS], l_s[AD_MERGE_GROUPS], m_s[AD_MERGE_GROUPS];
    pdl_launch_dependents();
    pdl_wait();
    const size_t th = blockIdx.x;                          // token * nh + head
    const float* src = part + th * n_splits * AD_ROW;
    const int col = threadIdx.x % AD_MERGE_COLS, grp = threadIdx.x / AD_MERGE_COLS;
    float m = -INFINITY;
    for (int s = grp; s < n_splits; s += AD_MERGE_GROUPS) m = fmaxf(m, src[(size_t)s * AD_ROW + AD_HD]);
    if (col == 0) m_s[grp] = m;
    __syncthreads();
    m = m_s[0];
#pragma unroll
    for (int w = 1; w < AD_MERGE_GROUPS; ++w) m = fmaxf(m, m_s[w]);
    float o = 0.f, l = 0.f;
#pragma unroll 4
    for (int s = grp; s < n_splits; s += AD_MERGE_GROUPS) {
        const float* p = src + (size_t)s * AD_ROW;
        const float wgt = (p[AD_HD] == -INFINITY) ? 0.f : exp2f(p[AD_HD] - m);
        if (col < AD_HD) o = fmaf(p[col], wgt, o);
        l = fmaf(p[AD_HD + 1], wgt, l);
    }
    o_s[grp][col] = o;
    if (col == 0) l_s[grp] = l;
    __syncthreads();
    if (grp == 0 && col < AD_HD) {
#pragma unroll
        for (int w = 1; w < AD_MERGE_GROUPS; ++w) { o += o_s[w][col]; l += l_s[w]; }
        out[th * AD_HD + col] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

extern "C" int pe_attention_decode_head_dim() { return AD_HD; }
extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }

// How many key ranges a launch over `max_context` keys uses: a function of the launch shape
// only, never of the sequences' lengths (the same launch is replayed as sequences grow).
extern "C" int pe_attention_decode_splits(int T, int nh, int nkv, int max_context, int* split_len_out) {
    const int G = nh / nkv, ctas = T * nkv * ((G + 15) / 16);
    int want = 148 * (AD_HD <= 64 ? 3 : 2) / ctas;            // one wave: what is resident at once (registers allow 3 or 2 CTAs an SM)
    const int most = (max_context + PE_PAGE - 1) / PE_PAGE;
    if (want > most) want = most;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    int split_len = ((max_context + want - 1) / want + PE_PAGE - 1) / PE_PAGE * PE_PAGE;
    if (split_len_out) *split_len_out = split_len;
    return (max_context + split_len - 1) / split_len;
}

extern "C" long long pe_attention_decode_scratch_bytes(int T, int nh, int nkv, int max_context) {
    const int n = pe_attention_decode_splits(T, nh, nkv, max_context, nullptr);
    return n > 1 ? (long long)T * nh * n * AD_ROW * 4 : 0;
}

extern "C" int pe_attention_decode(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                   const int* block_table, int table_stride, const int* tok_pos, const int* tok_row,
                                   int T, int nh, int nkv, int hd, int window, float scale, int max_context,
                                   void* scratch, void* stream) {
    if (T <= 0) return 0;
    if (hd != AD_HD || nkv <= 0 || nh % nkv || max_context <= 0 || q_stride % 8 || T > 65535) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return PE_ERR_UNSUPPORTED;
    int split_len = 0;
    const int n_splits = pe_attention_decode_splits(T, nh, nkv, max_context, &split_len);
    if (n_splits > 1 && !scratch) return PE_ERR_UNSUPPORTED;
    const int G = nh / nkv;
    const size_t smem = (size_t)AD_WARPS * 16 * AD_ROW * sizeof(float);
    static bool attr_set = false;
    if (smem > 48 * 1024 && !attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nkv * ((G + 15) / 16), n_splits);
    PE_TRY(pe_launch(attention_decode_kernel, grid, 32 * AD_WARPS, smem, s, 
        (const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_stride, tok_pos, tok_row,
        nh, nkv, window, scale * 1.4426950408889634f, split_len, n_splits, (float*)scratch, (bf16*)out));
    PE_LAUNCH_CHECK();
    if (n_splits > 1) {
        PE_TRY(pe_launch(attention_decode_merge_kernel, T * nh, AD_MERGE_GROUPS * AD_MERGE_COLS, 0, s, 
            (const float*)scratch, n_splits, (bf16*)out));
        PE_LAUNCH_CHECK();
    }
    return 0;
}
