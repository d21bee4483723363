// out[M, N] = A[M, K] . W[N, K]^T (+ bias[N]) on the CUDA cores: float32 multiply-add for
// every product, whatever the storage dtype of A and W.  This is the matrix product of the
// true 32-bit path (no tensor-core or reduced-precision mode is involved) and the fallback
// for operand dtypes that the tensor-core kernels do not take.
//
// The sum over k of one output element runs in increasing k, one fused multiply-add per k,
// whatever M is: a row's result does not depend on the rows beside it.
//
// pico-engine leaves these products to cuBLAS (src/pico_engine/model.py:177, 213, 223, 235, 164).
#include "common.cuh"

#define LS_BM 64
#define LS_BN 64
#define LS_BK 16

// epilogue: 0 store float32, 1 store bfloat16, 2 add into float32 (the residual stream)
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) linear_simt_kernel(const TA* A, const TW* W,
                                                          const void* bias, int bias_dtype,
                                                          void* out, int epilogue, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[LS_BK][LS_BM + 4];
    __shared__ float Ws[LS_BK][LS_BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * LS_BM, n0 = blockIdx.x * LS_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int lrow = tid >> 2, lk = (tid & 3) * 4;      // each thread loads 4 consecutive k of one row
    for (int k0 = 0; k0 < K; k0 += LS_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? to_f(A[(size_t)am * K + k]) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? to_f(W[(size_t)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < LS_BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 w = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_as_f(bias, bias_dtype, n);
            const size_t o = (size_t)m * N + n;
            if (epilogue == 0) ((float*)out)[o] = v;
            else if (epilogue == 1) ((bf16*)out)[o] = __float2bfloat16_rn(v);
            else ((float*)out)[o] += v;
        }
    }
}

extern "C" int pe_linear_simt(const void* A, int a_dtype, const void* W, int w_dtype, const void* bias, int bias_dtype,
                              void* out, int epilogue, int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || epilogue < 0 || epilogue > 2) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((N + LS_BN - 1) / LS_BN, (M + LS_BM - 1) / LS_BM);
    if (grid.y > 65535) return PE_ERR_UNSUPPORTED;
#define LS_GO(TA, TW) PE_TRY(pe_launch(linear_simt_kernel<TA, TW>, grid, 256, 0, s, (const TA*)A, (const TW*)W, bias, bias_dtype, out, epilogue, M, N, K))
    if (a_dtype == PE_F32 && w_dtype == PE_F32) LS_GO(float, float);
    else if (a_dtype == PE_BF16 && w_dtype == PE_BF16) LS_GO(bf16, bf16);
    else if (a_dtype == PE_BF16 && w_dtype == PE_F32) LS_GO(bf16, float);
    else if (a_dtype == PE_F32 && w_dtype == PE_BF16) LS_GO(float, bf16);
    else return PE_ERR_UNSUPPORTED;
#undef LS_GO
    PE_LAUNCH_CHECK();
    return 0;
}
