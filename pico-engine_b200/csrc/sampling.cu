// Choosing the next token of every row of float32 logits on the device: argmax, and
// temperature sampling with optional top-k and top-p, drawn by inverse CDF in index order
// from a counter-based uniform so that a sequence's draws depend on (seed, request, step)
// only, never on its neighbours in the batch.
//
// Semantics follow pico-engine's sampler (src/pico_engine/sampler.py:8-27): logits / temperature;
// top-k keeps every value >= the k-th largest (ties kept); top-p keeps a token iff the mass of
// the tokens ranked above it does not exceed top_p (the crossing token stays, the first token
// always stays); softmax; draw.  Two deliberate differences: the draw is seeded (the project
// uses torch's global generator, sampler.py:25), and logits that are bit-equal at the edge of
// the nucleus are kept or dropped together (a stable sort would split them by index).
#include "common.cuh"

#define SP_THREADS 1024

__device__ __forceinline__ unsigned int order_key(float f) {
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);     // monotonic: larger float, larger key
}

__device__ __forceinline__ double block_sum_d(double v, double* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum_d(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < nwarps ? scratch[lane] : 0.0;
        t = warp_sum_d(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ int block_sum_i(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = lane < nwarps ? scratch[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---------------------------------------------------------------- argmax (lowest index among equal maxima)
// Two stages so that one row of a large vocabulary is read by many blocks: each block reduces a
// chunk to one 64-bit word (ordered key of the value, then the complemented index, so that the
// maximum word is the largest value at its lowest index), a second kernel reduces the words.
#define AX_THREADS 256
#define AX_CHUNK 2048

__device__ __forceinline__ unsigned long long ax_pack(float v, int idx) {
    return ((unsigned long long)order_key(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)idx);
}
__device__ __forceinline__ unsigned long long ax_warp_max(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    return v;
}
__device__ __forceinline__ unsigned long long ax_block_max(unsigned long long v, unsigned long long* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = ax_warp_max(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarps ? scratch[lane] : 0ull;
        v = ax_warp_max(v);
    }
    return v;                                                 // valid in warp 0
}

__global__ void __launch_bounds__(AX_THREADS) argmax_partial_kernel(const float* logits, int V, int chunks,
                                                                    unsigned long long* part) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long scratch[32];
    const int b = blockIdx.y, c = blockIdx.x;
    const float* row = logits + (size_t)b * V;
    const int begin = c * AX_CHUNK, end = min(V, begin + AX_CHUNK);
    unsigned long long best = 0ull;
    for (int i = begin + threadIdx.x; i < end; i += AX_THREADS) {
        const unsigned long long p = ax_pack(row[i], i);
        best = p > best ? p : best;
    }
    best = ax_block_max(best, scratch);
    if (threadIdx.x == 0) part[(size_t)b * chunks + c] = best;
}

__global__ void __launch_bounds__(AX_THREADS) argmax_final_kernel(const unsigned long long* part, int chunks,
                                                                  int* out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long scratch[32];
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < chunks; i += AX_THREADS) {
        const unsigned long long p = part[(size_t)blockIdx.x * chunks + i];
        best = p > best ? p : best;
    }
    best = ax_block_max(best, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = (int)(0xFFFFFFFFu - (unsigned int)(best & 0xFFFFFFFFull));
}

extern "C" long long pe_argmax_scratch_bytes(int B, int V) { return (long long)B * ((V + AX_CHUNK - 1) / AX_CHUNK) * 8; }

extern "C" int pe_argmax(const float* logits, int* out, int B, int V, void* scratch, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || B > 65535 || !scratch) return PE_ERR_UNSUPPORTED;
    const int chunks = (V + AX_CHUNK - 1) / AX_CHUNK;
    cudaStream_t s = (cudaStream_t)stream;
    PE_TRY(pe_launch(argmax_partial_kernel, dim3(chunks, B), AX_THREADS, 0, s, logits, V, chunks, (unsigned long long*)scratch));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(argmax_final_kernel, B, AX_THREADS, 0, s, (const unsigned long long*)scratch, chunks, out));
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- the uniform of a draw
// splitmix64 finaliser of (seed, request, step); the top 24 bits make a float in [0, 1).
__host__ __device__ inline float draw_uniform(unsigned long long seed, unsigned long long request, unsigned long long step) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ULL + request * 0xBF58476D1CE4E5B9ULL +
                           step * 0x94D049BB133111EBULL + 0x2545F4914F6CDD1DULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

extern "C" float pe_draw_uniform(unsigned long long seed, unsigned long long request, unsigned long long step) {
    return draw_uniform(seed, request, step);
}

// ---------------------------------------------------------------- temperature / top-k / top-p sampling
__global__ void __launch_bounds__(SP_THREADS) sample_kernel(const float* logits, int* out, int V,
                                                            float temperature, int top_k, float top_p,
                                                            unsigned long long seed, const int* request,
                                                            const int* step) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    __shared__ double dscratch[33];
    __shared__ double seg_excl[SP_THREADS];
    __shared__ int found, last_kept;
    const int b = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)b * V;

    // 1. maximum of the scaled logits
    float mx = -INFINITY;
    for (int i = tid; i < V; i += SP_THREADS) mx = fmaxf(mx, row[i] / temperature);
    mx = block_max(mx, fscratch);

    // 2. top-k: the key of the k-th largest scaled logit, by radix selection
    unsigned int k_key = 0u;
    if (top_k > 0 && top_k < V) {
        unsigned int prefix = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = prefix | (1u << bit);
            int cnt = 0;
            for (int i = tid; i < V; i += SP_THREADS) cnt += order_key(row[i] / temperature) >= cand;
            if (block_sum_i(cnt, iscratch) >= top_k) prefix = cand;
        }
        k_key = prefix;
    }

    // 3. mass of what top-k kept
    double part = 0.0;
    for (int i = tid; i < V; i += SP_THREADS) {
        const float x = row[i] / temperature;
        if (order_key(x) >= k_key) part += (double)expf(x - mx);
    }
    const double mass_k = block_sum_d(part, dscratch);

    // 4. top-p: the smallest key whose mass strictly above it is <= top_p * mass_k
    unsigned int p_key = 0u;
    if (top_p < 1.0f) {
        const double limit = (double)top_p * mass_k;
        unsigned int prefix = 0u;            // becomes the largest key K with mass_above(K) > limit
        bool any_false = false;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = prefix | (1u << bit);
            double above = 0.0;
            for (int i = tid; i < V; i += SP_THREADS) {
                const float x = row[i] / temperature;
                const unsigned int key = order_key(x);
                if (key >= k_key && key > cand) above += (double)expf(x - mx);
            }
            if (block_sum_d(above, dscratch) > limit) { prefix = cand; any_false = true; }
        }
        if (!any_false) {                    // is mass_above(0) itself within the limit?
            p_key = (mass_k > limit) ? 1u : 0u;   // keys are never 0 for finite floats; 1 keeps everything
        } else {
            p_key = prefix + 1u;
        }
    }
    const unsigned int keep_key = k_key > p_key ? k_key : p_key;

    // 5. inverse CDF in index order: thread t owns the contiguous indices [t*seg, (t+1)*seg)
    const int seg = (V + SP_THREADS - 1) / SP_THREADS;
    const int i0 = min(V, tid * seg), i1 = min(V, i0 + seg);
    if (tid == 0) { found = 0x7fffffff; last_kept = -1; }
    __syncthreads();
    double mine = 0.0;
    int last = -1;
    for (int i = i0; i < i1; ++i) {
        const float x = row[i] / temperature;
        if (order_key(x) >= keep_key) { mine += (double)expf(x - mx); last = i; }
    }
    seg_excl[tid] = mine;
    if (last >= 0) atomicMax(&last_kept, last);
    __syncthreads();
    if (tid == 0) {                          // exclusive scan of the segment sums, in index order
        double run = 0.0;
        for (int t = 0; t < SP_THREADS; ++t) { const double v = seg_excl[t]; seg_excl[t] = run; run += v; }
        dscratch[0] = run;
    }
    __syncthreads();
    const double total = dscratch[0];
    const float u = draw_uniform(seed, (unsigned long long)request[b], (unsigned long long)step[b]);
    const double target = (double)u * total;
    double run = seg_excl[tid];
    if (run <= target && target < run + mine) {
        for (int i = i0; i < i1; ++i) {
            const float x = row[i] / temperature;
            if (order_key(x) >= keep_key) {
                run += (double)expf(x - mx);
                if (run > target) { atomicMin(&found, i); break; }
            }
        }
    }
    __syncthreads();
    // rounding may leave the target beyond the last kept token: that token is taken then
    if (tid == 0) out[b] = found != 0x7fffffff ? found : (last_kept < 0 ? 0 : last_kept);
}

extern "C" int pe_sample(const float* logits, int* out, int B, int V, float temperature, int top_k, float top_p,
                         unsigned long long seed, const int* request, const int* step, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !(temperature > 0.f)) return PE_ERR_UNSUPPORTED;
    PE_TRY(pe_launch(sample_kernel, B, SP_THREADS, 0, (cudaStream_t)stream, logits, out, V, temperature, top_k, top_p, seed, request, step));
    PE_LAUNCH_CHECK();
    return 0;
}
