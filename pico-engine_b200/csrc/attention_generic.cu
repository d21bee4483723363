// Softmax attention of any number of tokens over the paged key/value cache, for every head
// size up to 256 and either dtype: the attention of the true 32-bit path, and the one that
// takes the shapes the tensor-core kernels refuse.  One block per (token, query head).
//
// A query at position p of its sequence sees the keys lo..p of that sequence, lo = 0 or
// p - window + 1.  Keys are visited in increasing position in chunks of the block size that
// start at lo, so the arithmetic of one (sequence, position, head) is the same whether the
// token came in a long prompt, alone, or beside other sequences.
//
// Scores, softmax and the weighted sum are float32 (pico-engine: src/pico_engine/kernels.py:
// 108-125; its result is stored through float16 at kernels.py:126, which is not done here).
#include "common.cuh"

#define AG_THREADS 128
#define AG_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(AG_THREADS) attention_generic_kernel(
    const T* q, int q_stride, T* out, const T* k_pool,
    const T* v_pool, const int* block_table, int table_stride,
    const int* tok_pos, const int* tok_row, int nh, int nkv, int hd, int window,
    float scale) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float q_s[AG_MAX_HD];
    __shared__ float p_s[AG_THREADS];
    __shared__ long long base_s[AG_THREADS];
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = tok_pos[t];
    const int* table = block_table + (size_t)tok_row[t] * table_stride;
    const int kvh = h / (nh / nkv);
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int d = tid; d < hd; d += AG_THREADS) q_s[d] = to_f(qp[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;                       // dims tid and tid + AG_THREADS
    for (int c0 = lo; c0 <= pos; c0 += AG_THREADS) {
        const int j = c0 + tid;
        float s = -INFINITY;
        long long base = -1;
        if (j <= pos) {
            const int page = table[j / PE_PAGE];
            if (page >= 0) {
                base = ((long long)page * nkv + kvh) * PE_PAGE * hd + (long long)(j % PE_PAGE) * hd;
                const T* kp = k_pool + base;
                float dot = 0.f;
                for (int d = 0; d < hd; ++d) dot = fmaf(q_s[d], to_f(kp[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        p_s[tid] = p;
        base_s[tid] = base;
        l = l * alpha + block_sum(p, scratch);          // block_sum synchronises: p_s and base_s are visible after it
        m = m_new;
        acc0 *= alpha; acc1 *= alpha;
        const int n = min(AG_THREADS, pos - c0 + 1);
        for (int jj = 0; jj < n; ++jj) {
            const long long b = base_s[jj];
            if (b < 0) continue;
            const float pj = p_s[jj];
            const T* vp = v_pool + b;
            if (tid < hd) acc0 = fmaf(pj, to_f(vp[tid]), acc0);
            if (tid + AG_THREADS < hd) acc1 = fmaf(pj, to_f(vp[tid + AG_THREADS]), acc1);
        }
        __syncthreads();                                 // p_s and base_s are rewritten by the next chunk
    }
    T* op = out + ((size_t)t * nh + h) * hd;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    if (tid < hd) op[tid] = from_f<T>(acc0 * inv);
    if (tid + AG_THREADS < hd) op[tid + AG_THREADS] = from_f<T>(acc1 * inv);
}

extern "C" int pe_attention_generic(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                    int dtype, const int* block_table, int table_stride, const int* tok_pos,
                                    const int* tok_row, int T, int nh, int nkv, int hd, int window, float scale,
                                    void* stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > AG_MAX_HD || nkv <= 0 || nh % nkv || nh > 65535) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh);
    if (dtype == PE_F32)
        PE_TRY(pe_launch(attention_generic_kernel<float>, grid, AG_THREADS, 0, s, (const float*)q, q_stride, (float*)out,
            (const float*)k_pool, (const float*)v_pool, block_table, table_stride, tok_pos, tok_row, nh, nkv, hd, window, scale));
    else if (dtype == PE_BF16)
        PE_TRY(pe_launch(attention_generic_kernel<bf16>, grid, AG_THREADS, 0, s, (const bf16*)q, q_stride, (bf16*)out,
            (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_stride, tok_pos, tok_row, nh, nkv, hd, window, scale));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}
