// Tensor maps for TMA copies of boxes out of a row-major matrix, and the copy itself.
#pragma once
#include "common.cuh"
#include <cuda.h>

typedef CUresult (*pe_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, looked up through the runtime (the library is not linked against the driver).
inline pe_encode_tiled_fn pe_tensor_map_encoder() {
    static pe_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (pe_encode_tiled_fn)sym;
    }
    return fn;
}

// A [rows, cols] row-major matrix, loaded (or reduced into) in boxes of box_cols x box_rows with 128-byte swizzle; what a
// box holds beyond the matrix reads as zero.  `base` 16-byte aligned, the row pitch a multiple of 16 bytes.
inline int pe_tensor_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows, int box_cols, bool f32) {
    pe_encode_tiled_fn enc = pe_tensor_map_encoder();
    if (!enc) return PE_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * (f32 ? 4 : 2)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                           dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

// The box at column x (x times the element size a multiple of 16 bytes), row y into shared memory; its bytes complete on `bar`.
__device__ __forceinline__ void pe_tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
