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
// A row of a large vocabulary is read by many blocks (a chunk of SS_CHUNK logits each), in a few passes:
//
//   max     the largest scaled logit of the row (atomicMax on its ordered key)
//   select  the key of the k-th largest logit (top-k), then the smallest key whose mass strictly above it
//           is within top_p of the kept mass (top-p): a radix selection over the 32-bit ordered keys in three
//           levels of 11, 11 and 10 bits.  A pass adds, for the keys that share the prefix found so far, a
//           count and a mass per value of the level's bits into the row's histogram; the block of the row
//           that finishes last walks the histogram from the top, extends the prefix and clears the histogram.
//   draw    every block sums the kept mass of its chunk; the block of the row that finishes last finds the
//           chunk and then the index at which the running mass, in index order, passes uniform x total.
//
// Masses are exp(x - max) in 39-bit fixed point, summed as integers: sums do not depend on the order of the
// atomic additions, so the choice is the same from run to run and does not depend on the other rows.
// Plain temperature sampling is 2 launches, top-p 5, top-k and top-p 8, each over all rows.
#define SS_THREADS 256
#define SS_CHUNK 2048
#define SS_BINS 2048
#define SS_PER_THREAD (SS_CHUNK / SS_THREADS)

struct SsRow {                      // the state of one row between the passes; all zero between calls
    unsigned int max_key;           // ordered key of the largest scaled logit
    unsigned int ticket;            // blocks of the row that have finished the current pass
    unsigned int prefix;            // of the selection in progress: the key bits found so far
    unsigned int k_key, p_key;      // results of the selections (0: everything passes)
    unsigned int want;              // top-k: how many keys are still wanted at or below the prefix
    unsigned long long above;       // top-k and top-p: mass strictly above the prefix
    unsigned long long mass_k;      // mass of what top-k kept
    unsigned long long limit;       // top-p: top_p x mass_k
    unsigned long long pad;
};

__device__ __forceinline__ float key_value(unsigned int k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ unsigned long long fixed_mass(float x, float mx) {
    return __float2ull_rz(expf(x - mx) * 549755813888.0f);           // 2^39
}
__device__ __forceinline__ int ss_shift(int level) { return level == 0 ? 21 : (level == 1 ? 10 : 0); }
__device__ __forceinline__ int ss_bins(int level) { return level == 2 ? 1024 : 2048; }

// true in every thread of the last block of row b to arrive (all blocks' writes are visible to it)
__device__ __forceinline__ bool ss_last_block(SsRow* row, int blocks) {
    __shared__ int last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(&row->ticket, 1u);
        last = (t == (unsigned int)blocks - 1u);
        if (last) row->ticket = 0u;
    }
    __syncthreads();
    if (last) __threadfence();
    return last;
}

// Exclusive prefix sum of v over the threads of the block, in thread order; total: the sum of all.
// `scratch`: SS_THREADS words of shared memory (used between two barriers).
__device__ __forceinline__ unsigned long long ss_scan(unsigned long long v, unsigned long long* scratch,
                                                      unsigned long long& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    unsigned long long before = 0ull, all = 0ull;
#pragma unroll
    for (int w = 0; w < SS_THREADS / 32; ++w) {
        const unsigned long long t = scratch[w];
        if (w < warp) before += t;
        all += t;
    }
    total = all;
    __syncthreads();
    return before + inc - v;
}

// The sampler's settings as a kernel reads them.  A launch gives them by value; where it also gives `device`
// (four 32-bit words and a 64-bit seed, written by the host before the launch), those are read instead, so
// that a captured launch follows settings that change from call to call.
struct SsSettings { float temperature; int top_k; float top_p; int unused; unsigned long long seed; };
__device__ __forceinline__ SsSettings ss_settings(const SsSettings& by_value, const SsSettings* device) {
    return device ? *device : by_value;
}

__global__ void __launch_bounds__(SS_THREADS) sample_max_kernel(const float* logits, int V, const SsSettings given,
                                                                const SsSettings* device, SsRow* rows) {
    pdl_launch_dependents();
    pdl_wait();
    const float temperature = ss_settings(given, device).temperature;
    __shared__ float fscratch[33];
    const int b = blockIdx.y;
    const float* row = logits + (size_t)b * V;
    const int begin = blockIdx.x * SS_CHUNK, end = min(V, begin + SS_CHUNK);
    float mx = -INFINITY;
    for (int i = begin + threadIdx.x; i < end; i += SS_THREADS) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, fscratch);                            // division by a positive number keeps the order: divide the max only
    if (threadIdx.x == 0) atomicMax(&rows[b].max_key, order_key(mx / temperature));
}

// One level of a selection.  by_mass 0: top-k (the k-th largest key); 1: top-p.
__global__ void __launch_bounds__(SS_THREADS) sample_select_kernel(const float* logits, int V, const SsSettings given,
                                                                   const SsSettings* device, SsRow* rows, unsigned int* h_count,
                                                                   unsigned long long* h_mass, int by_mass, int level) {
    pdl_launch_dependents();
    pdl_wait();
    const SsSettings set = ss_settings(given, device);
    const float temperature = set.temperature, top_p = set.top_p;
    const int top_k = set.top_k;
    // per bin: count, and the mass as the sums of its low 20 and its high 19 bits (native 32-bit atomics;
    // 4096 terms of a chunk cannot overflow either)
    __shared__ unsigned int s_count[SS_BINS], s_lo[SS_BINS], s_hi[SS_BINS];
    __shared__ unsigned long long t_mass[SS_THREADS];
    __shared__ int chosen;
    const int b = blockIdx.y, tid = threadIdx.x;
    SsRow* st = rows + b;
    const float* row = logits + (size_t)b * V;
    const int shift = ss_shift(level), bins = ss_bins(level);
    const unsigned int prefix = level == 0 ? 0u : st->prefix, k_key = by_mass ? st->k_key : 0u;
    const int up = level == 0 ? 32 : ss_shift(level - 1);           // the bits above this level must equal the prefix
    const float mx = key_value(st->max_key);
    for (int i = tid; i < SS_BINS; i += SS_THREADS) { s_count[i] = 0u; s_lo[i] = 0u; s_hi[i] = 0u; }
    __syncthreads();
    const int begin = blockIdx.x * SS_CHUNK, end = min(V, begin + SS_CHUNK);
    for (int i = begin + tid; i < end; i += SS_THREADS) {
        const float x = row[i] / temperature;
        const unsigned int key = order_key(x);
        if (key < k_key) continue;
        if (up < 32 && (key >> up) != (prefix >> up)) continue;
        const unsigned int bin = (key >> shift) & (unsigned int)(bins - 1);
        const unsigned long long m = fixed_mass(x, mx);
        atomicAdd(&s_count[bin], 1u);
        if (m) { atomicAdd(&s_lo[bin], (unsigned int)(m & 0xFFFFFu)); atomicAdd(&s_hi[bin], (unsigned int)(m >> 20)); }
    }
    __syncthreads();
    unsigned int* gc = h_count + (size_t)b * SS_BINS;
    unsigned long long* gm = h_mass + (size_t)b * SS_BINS;
    for (int i = tid; i < bins; i += SS_THREADS)
        if (s_count[i]) { atomicAdd(&gc[i], s_count[i]); atomicAdd(&gm[i], ((unsigned long long)s_hi[i] << 20) + s_lo[i]); }
    if (!ss_last_block(st, gridDim.x)) return;

    // ---- the row's last block: walk the histogram from the top.  Thread t owns bins [t * per, (t + 1) * per).
    constexpr int per = SS_BINS / SS_THREADS;
    unsigned int c_mine = 0u, my_c[per];
    unsigned long long m_mine = 0ull, my_m[per];
#pragma unroll
    for (int i = 0; i < per; ++i) {
        const int bin = tid * per + i;
        my_c[i] = bin < bins ? gc[bin] : 0u; my_m[i] = bin < bins ? gm[bin] : 0ull;
    }
#pragma unroll
    for (int i = 0; i < per; ++i) { c_mine += my_c[i]; m_mine += my_m[i]; }
    if (tid == 0) chosen = -1;
    // the row's state is read by every thread before the barrier; the thread that finds the bin writes it after
    unsigned long long limit = st->limit, base = level == 0 ? 0ull : st->above;
    const unsigned long long mass_k = st->mass_k;
    unsigned int want = level == 0 ? (unsigned int)top_k : st->want;
    __syncthreads();
    // count and mass of the bins above this thread's: totals less the inclusive prefix sums
    unsigned long long c_total, m_total;
    const unsigned long long c_before = ss_scan((unsigned long long)c_mine, t_mass, c_total);
    const unsigned long long m_before = ss_scan(m_mine, t_mass, m_total);
    const unsigned int c_above = (unsigned int)(c_total - c_before - c_mine);
    const unsigned long long m_above = m_total - m_before - m_mine;
    if (by_mass && level == 0) {
        if (top_k <= 0 || top_k >= V) {                              // nothing was cut: what is kept is everything
            limit = (unsigned long long)((double)top_p * (double)m_total);
        } else {
            limit = (unsigned long long)((double)top_p * (double)mass_k);
        }
    }
    // top-k: the highest bin b with count(bins >= b) >= want.  top-p: the lowest bin b with base + mass(bins > b) <= limit.
    int mine = -1;
    unsigned int c_run = c_above;
    unsigned long long m_run = m_above;
    unsigned long long m_mine_bin = 0ull;                            // mass of the bin found
    if (!by_mass) {
#pragma unroll
        for (int i = per - 1; i >= 0; --i) {
            const int bin = tid * per + i;
            if (bin >= bins || mine >= 0) continue;
            if (c_run < want && c_run + my_c[i] >= want) { mine = bin; m_mine_bin = my_m[i]; continue; }
            c_run += my_c[i]; m_run += my_m[i];
        }
    } else {
#pragma unroll
        for (int i = per - 1; i >= 0; --i) {
            const int bin = tid * per + i;
            if (bin >= bins || mine >= 0) continue;
            // mass above this bin is m_run; the bin below it sees m_run + its mass
            const bool here = base + m_run <= limit;
            const bool below = bin > 0 && base + m_run + my_m[i] <= limit;
            if (here && !below) { mine = bin; continue; }
            m_run += my_m[i];
        }
    }
    if (mine >= 0) {                                                 // exactly one thread finds it
        chosen = mine;
        st->prefix = prefix | ((unsigned int)mine << shift);
        st->above = base + m_run;
        if (!by_mass) st->want = want - c_run;
        if (by_mass && level == 0) st->limit = limit;
        if (level == 2) {
            if (!by_mass) { st->k_key = prefix | (unsigned int)mine; st->mass_k = base + m_run + m_mine_bin; }
            else st->p_key = prefix | (unsigned int)mine;
            st->prefix = 0u; st->above = 0ull; st->want = 0u;
        }
    }
    __syncthreads();
    if (chosen < 0 && tid == 0) {                                    // top-k with fewer finite keys than k: keep everything
        st->prefix = 0u; st->above = 0ull; st->want = 0u;
        if (!by_mass) { st->k_key = 0u; st->mass_k = base + m_total; }
        else st->p_key = 0u;
    }
    for (int i = tid; i < SS_BINS; i += SS_THREADS) { gc[i] = 0u; gm[i] = 0ull; }      // the histogram is clear again
}

__global__ void __launch_bounds__(SS_THREADS) sample_draw_kernel(const float* logits, int* out, int V, const SsSettings given,
                                                                 const SsSettings* device, SsRow* rows,
                                                                 unsigned long long* chunk_mass, int* chunk_last,
                                                                 const int* request, const int* step) {
    pdl_launch_dependents();
    pdl_wait();
    const SsSettings set = ss_settings(given, device);
    const float temperature = set.temperature;
    const unsigned long long seed = set.seed;
    __shared__ unsigned long long seg[SS_THREADS];
    __shared__ unsigned long long s_total, s_before;
    __shared__ int s_chunk, s_found, s_last;
    const int b = blockIdx.y, tid = threadIdx.x, chunks = gridDim.x;
    SsRow* st = rows + b;
    const float* row = logits + (size_t)b * V;
    const float mx = key_value(st->max_key);
    const unsigned int keep = st->k_key > st->p_key ? st->k_key : st->p_key;

    // the kept mass of thread t's contiguous indices of chunk c, and the last kept index
    auto segment = [&](int c, int& last) {
        const int i0 = min(V, c * SS_CHUNK + tid * SS_PER_THREAD), i1 = min(V, i0 + SS_PER_THREAD);
        unsigned long long m = 0ull;
        for (int i = i0; i < i1; ++i) {
            const float x = row[i] / temperature;
            if (order_key(x) >= keep) { m += fixed_mass(x, mx); last = i; }
        }
        return m;
    };
    int last = -1;
    const unsigned long long own = segment(blockIdx.x, last);
    if (tid == 0) s_last = -1;
    __syncthreads();
    if (last >= 0) atomicMax(&s_last, last);
    unsigned long long chunk_total;
    ss_scan(own, seg, chunk_total);
    if (tid == 0) { chunk_mass[(size_t)b * chunks + blockIdx.x] = chunk_total; chunk_last[(size_t)b * chunks + blockIdx.x] = s_last; }
    if (!ss_last_block(st, chunks)) return;

    // ---- the row's last block: the first index at which the running kept mass, times 2^24, passes u24 x total
    const unsigned long long u24 = (unsigned long long)(draw_uniform(seed, (unsigned long long)request[b],
                                                                     (unsigned long long)step[b]) * 16777216.0f);
    // the chunk: thread t looks at chunks t, t + SS_THREADS, ...; a round scans the masses of SS_THREADS chunks
    if (tid == 0) { s_chunk = 0x7fffffff; s_found = 0x7fffffff; s_last = -1; s_total = 0ull; }
    __syncthreads();
    {
        unsigned long long total = 0ull;
        for (int c0 = 0; c0 < chunks; c0 += SS_THREADS) {
            const int c = c0 + tid;
            total += c < chunks ? chunk_mass[(size_t)b * chunks + c] : 0ull;
            if (c < chunks && chunk_last[(size_t)b * chunks + c] >= 0) atomicMax(&s_last, chunk_last[(size_t)b * chunks + c]);
        }
        unsigned long long all;
        ss_scan(total, seg, all);
        if (tid == 0) s_total = all;
        __syncthreads();
        const unsigned __int128 target = (unsigned __int128)u24 * s_total;
        unsigned long long before = 0ull;                            // mass of the rounds before this one
        for (int c0 = 0; c0 < chunks; c0 += SS_THREADS) {
            const int c = c0 + tid;
            const unsigned long long m = c < chunks ? chunk_mass[(size_t)b * chunks + c] : 0ull;
            unsigned long long round_total;
            const unsigned long long run = before + ss_scan(m, seg, round_total);      // mass before chunk c
            if (m && (((unsigned __int128)run) << 24) <= target && (((unsigned __int128)(run + m)) << 24) > target) {
                s_chunk = c; s_before = run;                         // exactly one chunk holds the crossing
            }
            before += round_total;
        }
    }
    __syncthreads();
    if (tid == 0 && s_chunk == 0x7fffffff) s_chunk = -1;
    __syncthreads();
    if (s_chunk >= 0) {
        int dummy = -1;
        const unsigned long long mine = segment(s_chunk, dummy);
        unsigned long long unused;
        unsigned long long run = s_before + ss_scan(mine, seg, unused);
        const unsigned __int128 target = (unsigned __int128)u24 * s_total;
        if (mine && (((unsigned __int128)run) << 24) <= target && (((unsigned __int128)(run + mine)) << 24) > target) {
            const int i0 = min(V, s_chunk * SS_CHUNK + tid * SS_PER_THREAD), i1 = min(V, i0 + SS_PER_THREAD);
            for (int i = i0; i < i1; ++i) {
                const float x = row[i] / temperature;
                if (order_key(x) >= keep) {
                    run += fixed_mass(x, mx);
                    if ((((unsigned __int128)run) << 24) > target) { atomicMin(&s_found, i); break; }
                }
            }
        }
    }
    __syncthreads();
    // everything the passes wrote is zero again (the scratch is laid out anew for other row counts and vocabularies)
    for (int c = tid; c < chunks; c += SS_THREADS) { chunk_mass[(size_t)b * chunks + c] = 0ull; chunk_last[(size_t)b * chunks + c] = 0; }
    if (tid == 0) {
        out[b] = s_found != 0x7fffffff ? s_found : (s_last < 0 ? 0 : s_last);
        st->max_key = 0u; st->k_key = 0u; st->p_key = 0u; st->mass_k = 0ull; st->limit = 0ull;
    }
}

extern "C" long long pe_sample_scratch_bytes(int B, int V) {
    const long long chunks = (V + SS_CHUNK - 1) / SS_CHUNK;
    return (long long)B * ((long long)sizeof(SsRow) + SS_BINS * 12ll + chunks * 12ll) + 256;
}

// `scratch`: pe_sample_scratch_bytes(B, V) bytes that are zero before the first call (every call leaves them zero).
// `settings`: null, or 24 bytes on the device (temperature as float, top_k as int, top_p as float, a word that is
// not read, the seed as 64 bits) that the kernels read instead of the scalar arguments; the scalar top_k and top_p
// still say which passes are launched (whether there is a cut by rank and one by mass), so they must agree on that.
extern "C" int pe_sample(const float* logits, int* out, int B, int V, float temperature, int top_k, float top_p,
                         unsigned long long seed, const int* request, const int* step, void* scratch, const void* settings,
                         void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !(temperature > 0.f) || B > 65535 || !scratch || (((uintptr_t)scratch) & 15) || (((uintptr_t)settings) & 7))
        return PE_ERR_UNSUPPORTED;
    SsSettings given = {temperature, top_k, top_p, 0, seed};
    const SsSettings* device = (const SsSettings*)settings;
    const int chunks = (V + SS_CHUNK - 1) / SS_CHUNK;
    SsRow* rows = (SsRow*)scratch;
    unsigned long long* h_mass = (unsigned long long*)(rows + B);
    unsigned long long* chunk_mass = h_mass + (size_t)B * SS_BINS;
    unsigned int* h_count = (unsigned int*)(chunk_mass + (size_t)B * chunks);
    int* chunk_last = (int*)(h_count + (size_t)B * SS_BINS);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(chunks, B);
    PE_TRY(pe_launch(sample_max_kernel, grid, SS_THREADS, 0, s, logits, V, given, device, rows));
    PE_LAUNCH_CHECK();
    const bool cut_k = top_k > 0 && top_k < V, cut_p = top_p < 1.0f;
    for (int by_mass = 0; by_mass < 2; ++by_mass) {
        if (by_mass ? !cut_p : !cut_k) continue;
        for (int level = 0; level < 3; ++level) {
            PE_TRY(pe_launch(sample_select_kernel, grid, SS_THREADS, 0, s, logits, V, given, device, rows, h_count, h_mass,
                             by_mass, level));
            PE_LAUNCH_CHECK();
        }
    }
    PE_TRY(pe_launch(sample_draw_kernel, grid, SS_THREADS, 0, s, logits, out, V, given, device, rows, chunk_mass, chunk_last,
                     request, step));
    PE_LAUNCH_CHECK();
    return 0;
}
