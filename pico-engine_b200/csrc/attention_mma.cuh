// Pieces shared by the tensor-core attention kernels (decode and prefill): the MMA, the
// register transpose that turns row-major value loads into B fragments, and the update of
// one warp's online-softmax state with a tile of 16 keys.
//
// Fragment conventions (lane = 4*g + t).  Scores of a 16-key tile are two m16n8 accumulators
// s[j][e]: row (e & 2 ? g + 8 : g), key j*8 + 2t + (e & 1).  The output accumulators are
// acc[c][r][e]: row as above, head-dimension column c*32 + t*8 + 2r + (e & 1).
// Q fragments qf[c][0/1] (rows g / g + 8) and key loads hold columns c*32 + t*8 .. +8 of a
// row, so both operands of S = Q.K^T see the head dimension in the same permuted order.
#pragma once
#include "common.cuh"

#define AM_HD PE_HEAD_DIM
#define AM_NCHUNK ((AM_HD + 31) / 32)

__device__ __forceinline__ void am_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned am_transpose(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ unsigned am_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// Queries, keys and values were written by kernels that may still have been running when this
// one started: they are read with plain coherent loads, never through the read-only path.
__device__ __forceinline__ uint4 am_ld16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Keys and values of one 16-key tile in registers: k[j][c] is the load of key j*8 + g,
// v[h][c] the load of value row h*8 + g, each columns c*32 + t*8 .. +8.
struct AmTile {
    uint4 k[2][AM_NCHUNK];
    uint4 v[2][AM_NCHUNK];
};

// base: element offset of the tile's first key row in the pool (rows are AM_HD apart).
__device__ __forceinline__ void am_load_tile(AmTile& tile, const bf16* k_pool,
                                             const bf16* v_pool, size_t base, int g, int t) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int c = 0; c < AM_NCHUNK; ++c) {
        const bool cin = c * 32 + t * 8 + 8 <= AM_HD;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const size_t off = base + (size_t)(j * 8 + g) * AM_HD + c * 32 + t * 8;
            tile.k[j][c] = cin ? am_ld16(k_pool + off) : zero;
            tile.v[j][c] = cin ? am_ld16(v_pool + off) : zero;
        }
    }
}

__device__ __forceinline__ void am_scores(float (&s)[2][4], const uint4 (&qf)[AM_NCHUNK][2], const AmTile& tile) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int c = 0; c < AM_NCHUNK; ++c) {
            am_mma(s[j], qf[c][0].x, qf[c][1].x, qf[c][0].y, qf[c][1].y, tile.k[j][c].x, tile.k[j][c].y);
            am_mma(s[j], qf[c][0].z, qf[c][1].z, qf[c][0].w, qf[c][1].w, tile.k[j][c].z, tile.k[j][c].w);
        }
    }
}

// s holds scaled scores in the log2 domain, -INFINITY where a key is not visible.  Updates the
// running max, the running (per-lane partial) sum and the output accumulators.
__device__ __forceinline__ void am_softmax_accumulate(float (&s)[2][4], float (&m_run)[2], float (&l_run)[2],
                                                      float (&acc)[AM_NCHUNK][4][4], const AmTile& tile) {
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) tmax[e >> 1] = fmaxf(tmax[e >> 1], s[j][e]);
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
        const float m_new = fmaxf(m_run[r], tmax[r]);
        alpha[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
    }
    float p[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p[j][e] = (s[j][e] == -INFINITY) ? 0.f : exp2f(s[j][e] - m_run[e >> 1]);
            l_run[e >> 1] += p[j][e];
        }
    const unsigned pa0 = am_pack(p[0][0], p[0][1]), pa1 = am_pack(p[0][2], p[0][3]);
    const unsigned pa2 = am_pack(p[1][0], p[1][1]), pa3 = am_pack(p[1][2], p[1][3]);
#pragma unroll
    for (int c = 0; c < AM_NCHUNK; ++c) {
        const unsigned lo_r[4] = {tile.v[0][c].x, tile.v[0][c].y, tile.v[0][c].z, tile.v[0][c].w};
        const unsigned hi_r[4] = {tile.v[1][c].x, tile.v[1][c].y, tile.v[1][c].z, tile.v[1][c].w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            acc[c][r][0] *= alpha[0]; acc[c][r][1] *= alpha[0];
            acc[c][r][2] *= alpha[1]; acc[c][r][3] *= alpha[1];
            am_mma(acc[c][r], pa0, pa1, pa2, pa3, am_transpose(lo_r[r]), am_transpose(hi_r[r]));
        }
    }
}
