// Embedding lookup, RMSNorm, SwiGLU and the rotary encoding fused with the write of keys
// and values into the paged cache.  All arithmetic is float32; only loads and stores
// convert.  The residual stream is float32 in both engine dtypes.
//
// pico-engine's counterparts are the Triton kernels _rmsnorm_fwd, _rope_fwd and
// _silu_mul_fwd (src/pico_engine/kernels.py:14-23, 37-47, 62-74), the torch gather at
// src/pico_engine/model.py:152 and the index_copy_ cache write at model.py:190-196.
#include "common.cuh"

// 1: kernels of this library may overlap their predecessor's tail (the default); 0: plain stream order.
extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* table, const int* ids, float* out,
                             int H, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);          // the host refuses such ids; never read outside the table
    const TW* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f(row[i]);
}

extern "C" int pe_embed(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int V,
                        void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == PE_F32) PE_TRY(pe_launch(embed_kernel<float>, T, 256, 0, s, (const float*)table, ids, out, H, V));
    else if (table_dtype == PE_BF16) PE_TRY(pe_launch(embed_kernel<bf16>, T, 256, 0, s, (const bf16*)table, ids, out, H, V));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// Token ids of a step that follows a step still in flight: ids[j] = prev[src[j]] where src[j] >= 0
// (the token that row src[j] of the step before chose, which the host has not seen yet);
// other ids stay as the host gave them.
__global__ void select_tokens_kernel(int* ids, const int* prev, const int* src, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n && src[j] >= 0) ids[j] = prev[src[j]];
}

extern "C" int pe_select_tokens(int* ids, const int* prev, const int* src, int n, void* stream) {
    if (n <= 0) return 0;
    PE_TRY(pe_launch(select_tokens_kernel, (n + 127) / 128, 128, 0, (cudaStream_t)stream, ids, prev, src, n));
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- RMSNorm
// One block per output row.  `rows_index` (may be null) picks the input row of each output
// row, so the final norm runs only on the rows whose logits are wanted.
__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* o, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<unsigned*>(&lo); v.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(o) = v;
}

__device__ __forceinline__ float4 load4_as_f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4_as_f(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// With ADD the row of y is first added to the row of x, which is written back: the residual sum
// that precedes the norm, in the same pass.  A thread keeps up to RN_KEEP groups of four elements in
// registers between the two passes and fetches their weights before the block-wide sum, so that
// the sum's latency hides the fetch; longer rows are read again.
#define RN_KEEP 4

template <typename TO, typename TY, bool ADD>
__global__ void rmsnorm_kernel(float* x, const TY* y, const int* rows_index,
                               const void* w, int w_dtype, float eps, TO* out, int H) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows_index ? rows_index[r] : r;
    float* xr = x + src * H;
    TO* o = out + (size_t)r * H;
    float ss = 0.f;
    if ((H & 3) == 0) {                                       // rows start on 16-byte boundaries
        float4* x4 = reinterpret_cast<float4*>(xr);
        const int n4 = H / 4;
        float4 v[RN_KEEP], wv[RN_KEEP];
#pragma unroll
        for (int k = 0; k < RN_KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                v[k] = x4[i];
                if (ADD) {
                    const float4 a = load4_as_f(y + src * H + 4 * i);
                    v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                    x4[i] = v[k];
                }
                ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss); ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
            }
        }
        for (int i = threadIdx.x + RN_KEEP * blockDim.x; i < n4; i += blockDim.x) {
            float4 u = x4[i];
            if (ADD) {
                const float4 a = load4_as_f(y + src * H + 4 * i);
                u.x += a.x; u.y += a.y; u.z += a.z; u.w += a.w;
                x4[i] = u;
            }
            ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
        }
#pragma unroll
        for (int k = 0; k < RN_KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) wv[k] = make_float4(load_as_f(w, w_dtype, 4 * i), load_as_f(w, w_dtype, 4 * i + 1),
                                            load_as_f(w, w_dtype, 4 * i + 2), load_as_f(w, w_dtype, 4 * i + 3));
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int k = 0; k < RN_KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) store4(o + 4 * i, v[k].x * rstd * wv[k].x, v[k].y * rstd * wv[k].y, v[k].z * rstd * wv[k].z, v[k].w * rstd * wv[k].w);
        }
        for (int i = threadIdx.x + RN_KEEP * blockDim.x; i < n4; i += blockDim.x) {
            const float4 u = x4[i];                           // this thread wrote it, if anyone did
            store4(o + 4 * i, u.x * rstd * load_as_f(w, w_dtype, 4 * i), u.y * rstd * load_as_f(w, w_dtype, 4 * i + 1),
                   u.z * rstd * load_as_f(w, w_dtype, 4 * i + 2), u.w * rstd * load_as_f(w, w_dtype, 4 * i + 3));
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float u = xr[i];
        if (ADD) { u += to_f(y[src * H + i]); xr[i] = u; }
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f<TO>(xr[i] * rstd * load_as_f(w, w_dtype, i));
}

// The same for many rows: a warp to a row, eight rows to a block, so that a step of thousands of rows is a few hundred
// blocks that never wait at a block-wide barrier (the sum of a row's squares is a warp's shuffle).  A lane keeps up
// to RW_KEEP groups of four elements between the two passes; a longer row is read again (from L2).
#define RW_KEEP 8
#define RW_WARPS 8

template <typename TO, typename TY, bool ADD>
__global__ void __launch_bounds__(32 * RW_WARPS) rmsnorm_rows_kernel(float* x, const TY* y, const void* w, int w_dtype, float eps,
                                                                     TO* out, int rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, r = blockIdx.x * RW_WARPS + (threadIdx.x >> 5);
    if (r >= rows) return;
    float4* x4 = reinterpret_cast<float4*>(x + (size_t)r * H);
    TO* o = out + (size_t)r * H;
    const int n4 = H / 4;
    float4 v[RW_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < RW_KEEP; ++k) {
        const int i = lane + 32 * k;
        if (i < n4) {
            v[k] = x4[i];
            if (ADD) {
                const float4 a = load4_as_f(y + (size_t)r * H + 4 * i);
                v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                x4[i] = v[k];
            }
            ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss); ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
        }
    }
    for (int i = lane + 32 * RW_KEEP; i < n4; i += 32) {
        float4 u = x4[i];
        if (ADD) {
            const float4 a = load4_as_f(y + (size_t)r * H + 4 * i);
            u.x += a.x; u.y += a.y; u.z += a.z; u.w += a.w;
            x4[i] = u;
        }
        ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < RW_KEEP; ++k) {
        const int i = lane + 32 * k;
        if (i < n4) store4(o + 4 * i, v[k].x * rstd * load_as_f(w, w_dtype, 4 * i), v[k].y * rstd * load_as_f(w, w_dtype, 4 * i + 1),
                           v[k].z * rstd * load_as_f(w, w_dtype, 4 * i + 2), v[k].w * rstd * load_as_f(w, w_dtype, 4 * i + 3));
    }
    for (int i = lane + 32 * RW_KEEP; i < n4; i += 32) {
        const float4 u = x4[i];                               // this lane wrote it, if anyone did
        store4(o + 4 * i, u.x * rstd * load_as_f(w, w_dtype, 4 * i), u.y * rstd * load_as_f(w, w_dtype, 4 * i + 1),
               u.z * rstd * load_as_f(w, w_dtype, 4 * i + 2), u.w * rstd * load_as_f(w, w_dtype, 4 * i + 3));
    }
}

template <typename TY, bool ADD>
static int rmsnorm_launch(float* x, const TY* y, const int* rows_index, const void* w, int w_dtype, float eps, void* out,
                          int out_dtype, int rows, int H, cudaStream_t s) {
    // many whole rows: a warp a row.  Measured inside a graph at 896 columns: level with a block a row at 2,048 rows
    // (3.7 against 4.2 us, with the residual sum 6.0 against 5.3 us), ahead at 8,192 (10.0 against 12.6, 17.5 against 19.2 us)
    if (!rows_index && rows >= 4096 && (H & 3) == 0 && H <= 8192) {
        const int blocks = (rows + RW_WARPS - 1) / RW_WARPS;
        if (out_dtype == PE_F32) PE_TRY(pe_launch(rmsnorm_rows_kernel<float, TY, ADD>, blocks, 32 * RW_WARPS, 0, s, x, y, w, w_dtype, eps, (float*)out, rows, H));
        else if (out_dtype == PE_BF16) PE_TRY(pe_launch(rmsnorm_rows_kernel<bf16, TY, ADD>, blocks, 32 * RW_WARPS, 0, s, x, y, w, w_dtype, eps, (bf16*)out, rows, H));
        else return PE_ERR_UNSUPPORTED;
        PE_LAUNCH_CHECK();
        return 0;
    }
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (out_dtype == PE_F32) PE_TRY(pe_launch(rmsnorm_kernel<float, TY, ADD>, rows, threads, 0, s, x, y, rows_index, w, w_dtype, eps, (float*)out, H));
    else if (out_dtype == PE_BF16) PE_TRY(pe_launch(rmsnorm_kernel<bf16, TY, ADD>, rows, threads, 0, s, x, y, rows_index, w, w_dtype, eps, (bf16*)out, H));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

extern "C" int pe_rmsnorm(const float* x, const int* rows_index, const void* w, int w_dtype, float eps, void* out,
                          int out_dtype, int rows, int H, void* stream) {
    if (rows <= 0) return 0;
    return rmsnorm_launch<float, false>(const_cast<float*>(x), (const float*)nullptr, rows_index, w, w_dtype, eps, out, out_dtype, rows, H,
                                        (cudaStream_t)stream);
}

// x += y (every row, in place), then out = norm(x) * w: the residual sum and the norm that follows it in one pass
extern "C" int pe_add_rmsnorm(float* x, const void* y, int y_dtype, const void* w, int w_dtype, float eps, void* out,
                              int out_dtype, int rows, int H, void* stream) {
    if (rows <= 0) return 0;
    if (y_dtype == PE_BF16) {
        if ((H & 3) == 0 && ((uintptr_t)y & 7)) return PE_ERR_UNSUPPORTED;
        return rmsnorm_launch<bf16, true>(x, (const bf16*)y, nullptr, w, w_dtype, eps, out, out_dtype, rows, H, (cudaStream_t)stream);
    }
    if (y_dtype == PE_F32) {
        if ((H & 3) == 0 && ((uintptr_t)y & 15)) return PE_ERR_UNSUPPORTED;
        return rmsnorm_launch<float, true>(x, (const float*)y, nullptr, w, w_dtype, eps, out, out_dtype, rows, H, (cudaStream_t)stream);
    }
    return PE_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- SwiGLU
// gu is [T, 2I]: gate in the first I columns, up in the last I.  out[t, i] = silu(gate) * up.
__device__ __forceinline__ float silu_mul(float g, float u) { return g * (1.0f / (1.0f + expf(-g))) * u; }

template <typename T>
__global__ void swiglu_kernel(const T* gu, T* out, int I, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx % I;
        out[idx] = from_f<T>(silu_mul(to_f(gu[t * 2 * I + i]), to_f(gu[t * 2 * I + I + i])));
    }
}

// I a multiple of 8: eight bfloat16 per thread and step with 16-byte loads and stores, two steps in
// flight.  The sigmoid uses the special-function unit's 2^x and reciprocal (relative error about
// 2^-22, far below the bfloat16 rounding of the result); the exact routines cost several times
// the memory time of this kernel.
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r * u;
}
__device__ __forceinline__ uint4 swiglu8(const uint4 g, const uint4 u) {
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 gf = __bfloat1622float2(g2[e]), uf = __bfloat1622float2(u2[e]);
        o2[e] = __floats2bfloat162_rn(silu_mul_fast(gf.x, uf.x), silu_mul_fast(gf.y, uf.y));
    }
    return o;
}
__global__ void swiglu_bf16x8_kernel(const bf16* gu, bf16* out, int I, size_t groups) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = I / 8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups; idx += 2 * stride) {
        const size_t idx1 = idx + stride;
        const bool two = idx1 < groups;
        const size_t t0 = idx / per_row, i0 = (idx % per_row) * 8, t1 = two ? idx1 / per_row : t0, i1 = two ? (idx1 % per_row) * 8 : i0;
        const uint4 g0 = *reinterpret_cast<const uint4*>(gu + t0 * 2 * I + i0), u0 = *reinterpret_cast<const uint4*>(gu + t0 * 2 * I + I + i0);
        const uint4 g1 = *reinterpret_cast<const uint4*>(gu + t1 * 2 * I + i1), u1 = *reinterpret_cast<const uint4*>(gu + t1 * 2 * I + I + i1);
        *reinterpret_cast<uint4*>(out + t0 * I + i0) = swiglu8(g0, u0);
        if (two) *reinterpret_cast<uint4*>(out + t1 * I + i1) = swiglu8(g1, u1);
    }
}

extern "C" int pe_swiglu(const void* gu, void* out, int dtype, int T, int I, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    if (dtype == PE_BF16 && I % 8 == 0 && !(((uintptr_t)gu | (uintptr_t)out) & 15)) {
        const size_t groups = total / 8, want = (groups + 511) / 512;      // two groups a thread
        const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
        PE_TRY(pe_launch(swiglu_bf16x8_kernel, blocks, 256, 0, s, (const bf16*)gu, (bf16*)out, I, groups));
        PE_LAUNCH_CHECK();
        return 0;
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == PE_F32) PE_TRY(pe_launch(swiglu_kernel<float>, blocks, 256, 0, s, (const float*)gu, (float*)out, I, total));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(swiglu_kernel<bf16>, blocks, 256, 0, s, (const bf16*)gu, (bf16*)out, I, total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- residual add
// x[t, :] += y[t, :] in float32 (y in either dtype): the epilogue of a library matrix product.
template <typename T>
__global__ void residual_add_kernel(float* x, const T* y, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] += to_f(y[i]);
}

// total a multiple of 4, both pointers aligned for 4-element accesses
template <typename T>
__global__ void residual_add_x4_kernel(float* x, const T* y, size_t groups) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        float4 a = *reinterpret_cast<float4*>(x + 4 * i);
        const float4 b = load4_as_f(y + 4 * i);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        *reinterpret_cast<float4*>(x + 4 * i) = a;
    }
}

extern "C" int pe_residual_add(float* x, const void* y, int y_dtype, long long total, void* stream) {
    if (total <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (total % 4 == 0 && !(((uintptr_t)x | (uintptr_t)y) & 15) && (y_dtype == PE_F32 || y_dtype == PE_BF16)) {
        const long long groups = total / 4, wantg = (groups + 255) / 256;
        const int blocksg = (int)(wantg < 148 * 16 ? wantg : 148 * 16);
        if (y_dtype == PE_F32) PE_TRY(pe_launch(residual_add_x4_kernel<float>, blocksg, 256, 0, s, x, (const float*)y, (size_t)groups));
        else PE_TRY(pe_launch(residual_add_x4_kernel<bf16>, blocksg, 256, 0, s, x, (const bf16*)y, (size_t)groups));
        PE_LAUNCH_CHECK();
        return 0;
    }
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (y_dtype == PE_F32) PE_TRY(pe_launch(residual_add_kernel<float>, blocks, 256, 0, s, x, (const float*)y, (size_t)total));
    else if (y_dtype == PE_BF16) PE_TRY(pe_launch(residual_add_kernel<bf16>, blocks, 256, 0, s, x, (const bf16*)y, (size_t)total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- bias add (library matrix product epilogue)
template <typename T>
__global__ void bias_add_kernel(T* y, const void* bias, int bias_dtype, int N, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        y[i] = from_f<T>(to_f(y[i]) + load_as_f(bias, bias_dtype, i % N));
}

extern "C" int pe_bias_add(void* y, int dtype, const void* bias, int bias_dtype, int M, int N, void* stream) {
    if (M <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)M * N;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == PE_F32) PE_TRY(pe_launch(bias_add_kernel<float>, blocks, 256, 0, s, (float*)y, bias, bias_dtype, N, total));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(bias_add_kernel<bf16>, blocks, 256, 0, s, (bf16*)y, bias, bias_dtype, N, total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- rotary encoding + cache write
// qkv is [T, (n_q + 2 n_kv) * hd]: query heads, key heads, value heads.  Query and key heads
// are rotated in place (pairs j, j + hd/2; cos/sin are float32 tables [positions, hd/2];
// null tables leave them as they are).  Rotated keys and the values are then written to the
// paged cache at (page of the token's sequence, position % PE_PAGE) when `store` is set.
// Pool layout: [page][kv head][PE_PAGE][hd].
template <typename T>
__global__ void rope_store_kernel(T* qkv, int n_q, int n_kv, int hd,
                                  const float* cos_t, const float* sin_t,
                                  const int* tok_pos, const int* tok_row,
                                  T* k_pool, T* v_pool,
                                  const int* block_table, int table_stride, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = hd >> 1;
    T* row = qkv + (size_t)t * (n_q + 2 * n_kv) * hd;
    size_t cache_base = 0;
    bool do_store = false;
    if (store) {
        const int page = block_table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
        do_store = page >= 0;
        cache_base = (size_t)page * n_kv * PE_PAGE * hd + (size_t)(pos % PE_PAGE) * hd;
    }
    const int n_rot = (n_q + n_kv) * half;
    for (int idx = threadIdx.x; idx < n_rot; idx += blockDim.x) {
        const int head = idx / half, j = idx % half;
        T* p = row + (size_t)head * hd;
        float a = to_f(p[j]), b = to_f(p[j + half]);
        if (cos_t) {
            const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
            const float ra = a * c - b * s, rb = a * s + b * c;
            a = ra; b = rb;
            p[j] = from_f<T>(a); p[j + half] = from_f<T>(b);
        }
        if (do_store && head >= n_q) {
            T* dst = k_pool + cache_base + (size_t)(head - n_q) * PE_PAGE * hd;
            dst[j] = from_f<T>(a); dst[j + half] = from_f<T>(b);
        }
    }
    if (do_store) {
        const T* v = row + (size_t)(n_q + n_kv) * hd;
        for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
            const int head = idx / hd, d = idx % hd;
            v_pool[cache_base + (size_t)head * PE_PAGE * hd + d] = v[idx];
        }
    }
}

// The same for bfloat16 with head sizes that are multiples of 16: eight elements per thread, 16-byte accesses.
__global__ void rope_store_bf16x8_kernel(bf16* qkv, int n_q, int n_kv, int hd, const float* cos_t, const float* sin_t,
                                         const int* tok_pos, const int* tok_row, bf16* k_pool, bf16* v_pool,
                                         const int* block_table, int table_stride, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = hd >> 1, groups = half >> 3;               // groups of 8 pairs per head
    bf16* row = qkv + (size_t)t * (n_q + 2 * n_kv) * hd;
    size_t cache_base = 0;
    bool do_store = false;
    if (store) {
        const int page = block_table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
        do_store = page >= 0;
        cache_base = (size_t)page * n_kv * PE_PAGE * hd + (size_t)(pos % PE_PAGE) * hd;
    }
    for (int idx = threadIdx.x; idx < (n_q + n_kv) * groups; idx += blockDim.x) {
        const int head = idx / groups, j = (idx % groups) * 8;
        bf16* p = row + (size_t)head * hd;
        uint4 lo = *reinterpret_cast<const uint4*>(p + j), hi = *reinterpret_cast<const uint4*>(p + j + half);
        if (cos_t) {
            const float* cp = cos_t + (size_t)pos * half + j;
            const float* sp = sin_t + (size_t)pos * half + j;
            const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(l2[e]), b = __bfloat1622float2(h2[e]);
                l2[e] = __floats2bfloat162_rn(a.x * c[2 * e] - b.x * sn[2 * e], a.y * c[2 * e + 1] - b.y * sn[2 * e + 1]);
                h2[e] = __floats2bfloat162_rn(a.x * sn[2 * e] + b.x * c[2 * e], a.y * sn[2 * e + 1] + b.y * c[2 * e + 1]);
            }
            *reinterpret_cast<uint4*>(p + j) = lo;
            *reinterpret_cast<uint4*>(p + j + half) = hi;
        }
        if (do_store && head >= n_q) {
            bf16* dst = k_pool + cache_base + (size_t)(head - n_q) * PE_PAGE * hd;
            *reinterpret_cast<uint4*>(dst + j) = lo;
            *reinterpret_cast<uint4*>(dst + j + half) = hi;
        }
    }
    if (do_store) {
        const bf16* v = row + (size_t)(n_q + n_kv) * hd;
        for (int idx = threadIdx.x; idx < n_kv * hd / 8; idx += blockDim.x) {
            const int head = (idx * 8) / hd, d = (idx * 8) % hd;
            *reinterpret_cast<uint4*>(v_pool + cache_base + (size_t)head * PE_PAGE * hd + d) = *reinterpret_cast<const uint4*>(v + idx * 8);
        }
    }
}

extern "C" int pe_rope_store(void* qkv, int dtype, int T, int n_q, int n_kv, int hd, const float* cos_t,
                             const float* sin_t, const int* tok_pos, const int* tok_row, void* k_pool, void* v_pool,
                             const int* block_table, int table_stride, int store, void* stream) {
    if (T <= 0) return 0;
    if (hd % 2) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32)
        PE_TRY(pe_launch(rope_store_kernel<float>, T, 256, 0, s, (float*)qkv, n_q, n_kv, hd, cos_t, sin_t, tok_pos, tok_row,
                                                    (float*)k_pool, (float*)v_pool, block_table, table_stride, store));
    else if (dtype == PE_BF16 && hd % 16 == 0 && !(((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15))
        PE_TRY(pe_launch(rope_store_bf16x8_kernel, T, 128, 0, s, (bf16*)qkv, n_q, n_kv, hd, cos_t, sin_t, tok_pos, tok_row,
                         (bf16*)k_pool, (bf16*)v_pool, block_table, table_stride, store));
    else if (dtype == PE_BF16)
        PE_TRY(pe_launch(rope_store_kernel<bf16>, T, 256, 0, s, (bf16*)qkv, n_q, n_kv, hd, cos_t, sin_t, tok_pos, tok_row,
                                                   (bf16*)k_pool, (bf16*)v_pool, block_table, table_stride, store));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}
