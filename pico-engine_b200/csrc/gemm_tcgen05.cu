// out = A[M, K] . W[N, K]^T for more than 16 rows (prompts, larger decode batches), bfloat16
// operands, on the 5th-generation tensor cores: tcgen05.mma with both operands in shared memory
// and float32 accumulators in tensor memory, fused with what follows the product in a decoder layer.
//
// A CTA is persistent: it takes output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... and keeps two
// accumulators in tensor memory, so that the epilogue of one tile runs while the tensor core works on the
// next one.
//
//   warp 0     producer: TMA tiled loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the two operand
//              tiles of a 64-wide k block into a ring of stages; the tiles of W of the first stages are
//              asked for before the kernel waits for its predecessor (no kernel writes weights)
//   warp 1     allocates tensor memory; one lane issues the tcgen05.mma of a stage (K = 16 each) and commits
//              them to the stage's "empty" barrier, the last of a tile to the accumulator's "full" barrier
//   warps 2-17 epilogue: four warps to each quarter of the accumulator's lanes, taking its 32-column chunks in turn
//              (a warp issues an instruction every 6 to 8 cycles here, so a scheduler needs several of them to
//              keep up with the tensor core): tcgen05.ld of 32 columns at a time, then one of
//                STORE   out[M, N] = acc + bias, bfloat16
//                ACCUM   x[M, N] += acc, float32 (the residual sum): a TMA reduction from shared memory
//                        (many rows) or red.global.add (few rows), so x is not read by the SM
//                SWIGLU  act[M, I] = silu(gate) * up, gate and up being rows i and I + i of W
//                ROPE    rows of W are query, key and value heads: add bias, rotate query and key heads by
//                        position, write queries to out and keys and values into the paged cache
//
// Two orientations.  Many rows: the 128 lanes of the accumulator are 128 rows of A (tokens), its columns
// BN rows of W.  Few rows (up to 128 a tile, "swapped"): the lanes are 128 rows of W and the columns the
// tokens, so a handful of sequences still fills the tensor core's M side and the weights stream once.
//
// Every mbarrier wait is bounded by the clock; a wait that runs out sets *status to 2 and a flag in shared
// memory that makes every other role leave its loop; tensor memory is freed and the CTA returns.
//
// pico-engine leaves these products to cuBLAS under fp16 autocast and runs bias, rotation, cache write,
// residual and activation as separate launches (src/pico_engine/model.py:177-235, kernels.py:37-87).
#include "common.cuh"
#include "tensor_map.cuh"

#define GT_BK 64
#define GT_EPI_WARPS 16
#define GT_EPI_THREADS (32 * GT_EPI_WARPS)
#define GT_THREADS (64 + GT_EPI_THREADS)  // producer warp, MMA warp, the epilogue warps
#define GT_WAIT_CYCLES 2000000000ll
#define GT_SMEM_BYTES (227 * 1024 - 2048) // dynamic shared memory of a CTA: the operand ring and the epilogue's staging

enum { GT_STORE = 0, GT_ACCUM = 1, GT_SWIGLU = 2, GT_ROPE = 3 };

struct GtArgs {
    void* out; const void* bias; int bias_dtype;
    int M, N, K;           // M rows of A; N rows of W (SWIGLU: N = 2 I)
    int I;                 // SWIGLU: columns of the result
    int tiles_m, tiles;    // tiles along the rows of A; all tiles (tile t: m = t % tiles_m, n = t / tiles_m)
    // ROPE
    int n_q, n_kv, hd;
    const float* cos_t; const float* sin_t;
    const int* tok_pos; const int* tok_row;
    bf16* k_pool; bf16* v_pool; const int* block_table; int table_stride; int store;
};

__device__ __forceinline__ unsigned gt_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// true when the phase with this parity has completed; false when the wait ran out or another role gave up
__device__ __forceinline__ bool gt_wait(unsigned bar, unsigned parity, const volatile int* abort_flag) {
    unsigned done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    const long long deadline = clock64() + GT_WAIT_CYCLES;
    for (unsigned spins = 1;; ++spins) {
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((spins & 63u) == 0 && (*abort_flag || clock64() > deadline)) return false;
    }
}
__device__ __forceinline__ void gt_tma_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// x[...] += the float32 box in shared memory, done by the memory system
__device__ __forceinline__ void gt_tma_reduce_add_2d(const CUtensorMap* map, int x, int y, unsigned src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
// K-major operand tile [rows][64 bfloat16] in 128-byte swizzle: 8-row groups are 1024 bytes apart
__device__ __forceinline__ unsigned long long gt_desc(unsigned smem_addr) {
    return (unsigned long long)((smem_addr >> 4) & 0x3FFFu) | ((unsigned long long)(1024u >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void gt_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void gt_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gt_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ unsigned gt_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float gt_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// silu(g) * u with g and u rounded to bfloat16 first, as the unfused path stores them
__device__ __forceinline__ float gt_swiglu(float g, float u) {
    g = gt_round(g); u = gt_round(u);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r * u;
}
// the bias of the 32 columns from n on (N is a multiple of 8: groups of 8 are inside or outside), or zeros
__device__ __forceinline__ void gt_bias32(const GtArgs& p, int n, float (&b)[32]) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        if (p.bias && n + i < p.N) {
            if (p.bias_dtype == PE_BF16) {
                const uint4 v = *reinterpret_cast<const uint4*>((const bf16*)p.bias + n + i);
                const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(v2[e]); b[i + 2 * e] = f.x; b[i + 2 * e + 1] = f.y; }
            } else {
                const float4 v0 = *reinterpret_cast<const float4*>((const float*)p.bias + n + i);
                const float4 v1 = *reinterpret_cast<const float4*>((const float*)p.bias + n + i + 4);
                b[i] = v0.x; b[i + 1] = v0.y; b[i + 2] = v0.z; b[i + 3] = v0.w; b[i + 4] = v1.x; b[i + 5] = v1.y; b[i + 6] = v1.z; b[i + 7] = v1.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) b[i + e] = 0.f;
        }
    }
}
// all epilogue threads (GT_EPI_THREADS = 512) meet and learn whether every one of them passed `ok`
__device__ __forceinline__ bool gt_epilogue_all(bool ok) {
    unsigned r;
    asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 q, %1, 0;\n barrier.red.and.pred p, 1, 512, q;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(r) : "r"((unsigned)ok) : "memory");
    return r != 0;
}
__device__ __forceinline__ void gt_epilogue_sync() { asm volatile("barrier.sync 1, 512;" ::: "memory"); }

// What the epilogue warps turn their results through: ACCUM a 4 KB box a warp, ROPE a tile of 128 tokens x 128 features.
constexpr unsigned gt_staging_bytes(int epi) { return epi == GT_ACCUM ? GT_EPI_WARPS * 4096u : epi == GT_ROPE ? 32768u : 0u; }
constexpr int gt_stages(unsigned stage_bytes, int epi) {
    return (int)((GT_SMEM_BYTES - 1024u - gt_staging_bytes(epi)) / stage_bytes) > 8 ? 8 : (int)((GT_SMEM_BYTES - 1024u - gt_staging_bytes(epi)) / stage_bytes);
}
constexpr int gt_pow2_cols(int c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : c <= 256 ? 256 : 512; }

// The results of a tile as bfloat16 [token][128 features] in shared memory (a row is 256 bytes; the 16-byte
// chunk c of token j lies at chunk c ^ (j & 7), which keeps both the writes of a warp and the reads below
// free of bank conflicts): rotate the halves of query and key heads and send every head where it belongs.
__device__ __forceinline__ void gt_rope_scatter(const GtArgs& p, const unsigned char* staging, int tokens, int m0, int n0, int tid) {
    const int hd = p.hd, half = hd >> 1, groups = hd >> 4;           // groups of 8 pairs in a head
    const int per_token = (128 / hd) * groups;                        // = 8
    for (int idx = tid; idx < tokens * per_token; idx += GT_EPI_THREADS) {
        const int j = idx / per_token, rest = idx % per_token, hl = rest / groups, g = rest % groups;
        const int m = m0 + j, head = n0 / hd + hl, d = g * 8;
        if (m >= p.M || head >= p.n_q + 2 * p.n_kv) continue;
        const int c_lo = hl * (hd >> 3) + g, c_hi = c_lo + groups;
        uint4 lo = *reinterpret_cast<const uint4*>(staging + j * 256 + ((c_lo ^ (j & 7)) << 4));
        uint4 hi = *reinterpret_cast<const uint4*>(staging + j * 256 + ((c_hi ^ (j & 7)) << 4));
        const int pos = p.tok_pos[m];
        if (head < p.n_q + p.n_kv && p.cos_t) {
            const float* cp = p.cos_t + (size_t)pos * half + d;
            const float* sp = p.sin_t + (size_t)pos * half + d;
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
        }
        bf16* dst;
        if (head < p.n_q) {
            dst = (bf16*)p.out + (size_t)m * p.n_q * hd + (size_t)head * hd;
        } else {
            if (!p.store) continue;
            const int page = p.block_table[(size_t)p.tok_row[m] * p.table_stride + pos / PE_PAGE];
            if (page < 0) continue;
            const bool is_k = head < p.n_q + p.n_kv;
            const int kvh = head - p.n_q - (is_k ? 0 : p.n_kv);
            dst = (is_k ? p.k_pool : p.v_pool) + (((size_t)page * p.n_kv + kvh) * PE_PAGE + (pos % PE_PAGE)) * hd;
        }
        *reinterpret_cast<uint4*>(dst + d) = lo;
        *reinterpret_cast<uint4*>(dst + d + half) = hi;
    }
}

// The epilogue of one tile for one warp: its quarter of the accumulator's lanes, every fourth 32-column chunk.
template <bool SWAP, int BN, int EPI>
__device__ __forceinline__ void gt_epilogue_tile(const GtArgs& p, const CUtensorMap* map_out, unsigned taddr, int m0, int n0,
                                                 int quarter, int turn, int lane, unsigned char* staging, unsigned char* box,
                                                 int& staged) {
    if (!SWAP) {
        const int row = m0 + quarter * 32 + lane;           // this lane's token
        if (EPI == GT_SWIGLU) {
#pragma unroll 1
            for (int c = 32 * turn; c < 128; c += 32 * (GT_EPI_WARPS / 4)) {
                if (n0 + c >= p.I) break;
                float gate[32], up[32];
                gt_ld32(taddr + c, gate);
                gt_ld32(taddr + 128 + c, up);
                if (row < p.M) {
                    bf16* o = (bf16*)p.out + (size_t)row * p.I + n0 + c;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (n0 + c + i < p.I) {             // I is a multiple of 8
                            unsigned w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                w[e] = gt_pack(gt_swiglu(gate[i + 2 * e], up[i + 2 * e]), gt_swiglu(gate[i + 2 * e + 1], up[i + 2 * e + 1]));
                            *reinterpret_cast<uint4*>(o + i) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        } else if (EPI == GT_STORE) {
#pragma unroll 1
            for (int c = 32 * turn; c < BN; c += 32 * (GT_EPI_WARPS / 4)) {
                if (n0 + c >= p.N) break;
                float acc[32], bias[32];
                gt_bias32(p, n0 + c, bias);
                gt_ld32(taddr + c, acc);
                if (row < p.M) {
                    bf16* o = (bf16*)p.out + (size_t)row * p.N + n0 + c;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (n0 + c + i < p.N) {             // N is a multiple of 8
                            unsigned w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) w[e] = gt_pack(acc[i + 2 * e] + bias[i + 2 * e], acc[i + 2 * e + 1] + bias[i + 2 * e + 1]);
                            *reinterpret_cast<uint4*>(o + i) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        } else if (EPI == GT_ACCUM) {
            // Into the float32 residual stream: the warp lays its 32 rows x 32 columns out in shared memory as
            // the 128-byte-swizzled box of a TMA reduction, which adds them to x in memory.
            if (m0 + quarter * 32 < p.M) {
#pragma unroll 1
                for (int c = 32 * turn; c < BN; c += 32 * (GT_EPI_WARPS / 4)) {
                    if (n0 + c >= p.N) break;
                    float acc[32];
                    gt_ld32(taddr + c, acc);
                    if (staged) {                           // the box sent last has been read
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        __syncwarp();
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                            make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        gt_tma_reduce_add_2d(map_out, n0 + c, m0 + quarter * 32, gt_smem(box));
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    ++staged;
                }
            }
        } else {                                            // GT_ROPE: bfloat16(acc + bias) into the staging, by token
#pragma unroll 1
            for (int c = 32 * turn; c < 128; c += 32 * (GT_EPI_WARPS / 4)) {
                float acc[32], bias[32];
                gt_bias32(p, n0 + c, bias);
                gt_ld32(taddr + c, acc);
                const int j = quarter * 32 + lane;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    unsigned w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) w[e] = gt_pack(acc[i + 2 * e] + bias[i + 2 * e], acc[i + 2 * e + 1] + bias[i + 2 * e + 1]);
                    *reinterpret_cast<uint4*>(staging + j * 256 + ((((c + i) >> 3) ^ (j & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    } else {
        const int n = n0 + quarter * 32 + lane;             // this lane's feature (row of W)
        if (EPI == GT_SWIGLU) {
#pragma unroll 1
            for (int c = 32 * turn; c < BN; c += 32 * (GT_EPI_WARPS / 4)) {
                if (m0 + c >= p.M) break;
                float gate[32], up[32];
                gt_ld32(taddr + c, gate);
                gt_ld32(taddr + BN + c, up);
                if (n < p.I) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (m0 + c + j < p.M) ((bf16*)p.out)[(size_t)(m0 + c + j) * p.I + n] = __float2bfloat16_rn(gt_swiglu(gate[j], up[j]));
                }
            }
        } else if (EPI == GT_ROPE) {
            const float b = (p.bias && n < p.N) ? load_as_f(p.bias, p.bias_dtype, n) : 0.f;
            const int f = quarter * 32 + lane;
#pragma unroll 1
            for (int c = 32 * turn; c < BN; c += 32 * (GT_EPI_WARPS / 4)) {
                if (m0 + c >= p.M) break;
                float acc[32];
                gt_ld32(taddr + c, acc);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    *reinterpret_cast<bf16*>(staging + (c + j) * 256 + (((f >> 3) ^ ((c + j) & 7)) << 4) + (f & 7) * 2) = __float2bfloat16_rn(acc[j] + b);
            }
        } else {
            const float b = (EPI == GT_STORE && p.bias && n < p.N) ? load_as_f(p.bias, p.bias_dtype, n) : 0.f;
#pragma unroll 1
            for (int c = 32 * turn; c < BN; c += 32 * (GT_EPI_WARPS / 4)) {
                if (m0 + c >= p.M) break;
                float acc[32];
                gt_ld32(taddr + c, acc);
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (m0 + c + j < p.M) {
                            const size_t o = (size_t)(m0 + c + j) * p.N + n;
                            if (EPI == GT_STORE) ((bf16*)p.out)[o] = __float2bfloat16_rn(acc[j] + b);
                            else atomicAdd((float*)p.out + o, acc[j]);      // the only sum into this element: a reduction without a read
                        }
                    }
                }
            }
        }
    }
}

// SWAP false: A operand = 128 rows of the activations, B operand = BN rows of W (SWIGLU: 128 gate rows and
//             the 128 up rows that match them), accumulator lane = token, column = feature.
// SWAP true:  A operand = 128 rows of W (SWIGLU: a gate tile and an up tile, each with an accumulator of its
//             own), B operand = BN rows of the activations, accumulator lane = feature, column = token.
template <bool SWAP, int BN, int EPI>
__global__ void __launch_bounds__(GT_THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_act,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_out,
                                                                  const GtArgs p, int* status) {
    constexpr int NA = (SWAP && EPI == GT_SWIGLU) ? 2 : 1;                 // accumulators (tiles of W) of a tile
    constexpr unsigned A_BYTES = NA * 128 * GT_BK * 2, B_BYTES = BN * GT_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int STAGES = gt_stages(STAGE_BYTES, EPI);
    constexpr int ACC_COLS = NA * BN;                                      // columns of one accumulator buffer
    constexpr int TMEM_COLS = gt_pow2_cols(2 * ACC_COLS);
    constexpr int OUT_COLS = (!SWAP && EPI == GT_SWIGLU) ? 128 : BN;       // not swapped: result columns of a tile
    extern __shared__ __align__(1024) unsigned char gt_mem[];              // [stage][A tile | B tile], then the staging
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.K + GT_BK - 1) / GT_BK;
    const unsigned stage0 = (gt_smem(gt_mem) + 1023u) & ~1023u;            // 1024-byte aligned, as the swizzle needs
    unsigned char* const staging = gt_mem + (stage0 - gt_smem(gt_mem)) + STAGES * STAGE_BYTES;
    const volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&full_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&empty_bar[s])) : "memory");
        }
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&acc_full[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gt_smem(&acc_empty[b])), "r"(GT_EPI_WARPS) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"((unsigned)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_base_s;
    // Only now may the next kernel of the stream be scheduled: if it came earlier, took tensor memory on this SM
    // and then waited for this grid to end, a CTA of this grid that still had to allocate would wait for it in turn.
    pdl_launch_dependents();

    // tile t of this CTA: first row of A and first row of W (SWIGLU: of the gate rows)
    auto tile_m0 = [&](int t) { return (t % p.tiles_m) * (SWAP ? BN : 128); };
    auto tile_n0 = [&](int t) { return (t / p.tiles_m) * (SWAP ? 128 : OUT_COLS); };

    if (warp == 0) {
        if (lane == 0) {                                            // ---------------- producer
            const int my_tiles = ((int)blockIdx.x < p.tiles) ? (p.tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
            const long long total = (long long)my_tiles * k_blocks;
            auto load_w = [&](long long it) {
                const int t = (int)blockIdx.x + (int)(it / k_blocks) * (int)gridDim.x, kb = (int)(it % k_blocks), s = (int)(it % STAGES);
                const unsigned bar = gt_smem(&full_bar[s]), dst = stage0 + s * STAGE_BYTES;
                const int n0 = tile_n0(t);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STAGE_BYTES) : "memory");
                if (SWAP) {
                    gt_tma_2d(dst, &map_w, kb * GT_BK, n0, bar);
                    if (NA == 2) gt_tma_2d(dst + 128 * GT_BK * 2, &map_w, kb * GT_BK, p.I + n0, bar);
                } else if (EPI == GT_SWIGLU) {
                    gt_tma_2d(dst + A_BYTES, &map_w, kb * GT_BK, n0, bar);                         // gate rows
                    gt_tma_2d(dst + A_BYTES + 128 * GT_BK * 2, &map_w, kb * GT_BK, p.I + n0, bar);   // the matching up rows
                } else {
#pragma unroll
                    for (int r = 0; r < BN; r += 128) gt_tma_2d(dst + A_BYTES + r * GT_BK * 2, &map_w, kb * GT_BK, n0 + r, bar);
                }
            };
            auto load_act = [&](long long it) {
                const int t = (int)blockIdx.x + (int)(it / k_blocks) * (int)gridDim.x, kb = (int)(it % k_blocks), s = (int)(it % STAGES);
                gt_tma_2d(stage0 + s * STAGE_BYTES + (SWAP ? A_BYTES : 0u), &map_act, kb * GT_BK, tile_m0(t), gt_smem(&full_bar[s]));
            };
            const long long ahead = total < STAGES ? total : STAGES;
            for (long long it = 0; it < ahead; ++it) load_w(it);     // weights: nothing to wait for
            pdl_wait();
            for (long long it = 0; it < ahead; ++it) load_act(it);
            for (long long it = ahead; it < total; ++it) {
                const int s = (int)(it % STAGES);
                if (!gt_wait(gt_smem(&empty_bar[s]), (unsigned)((it / STAGES) - 1) & 1u, abort_flag)) { atomicExch(status, 2); abort_s = 1; break; }
                load_w(it);
                load_act(it);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                            // ---------------- MMA issuer
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = BN, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
            long long it = 0;
            bool ok = true;
            for (int t = blockIdx.x, lt = 0; t < p.tiles && ok; t += gridDim.x, ++lt) {
                const int buf = lt & 1;
                if (!gt_wait(gt_smem(&acc_empty[buf]), (unsigned)((lt >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned acc = tmem + (unsigned)(buf * ACC_COLS);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    if (!gt_wait(gt_smem(&full_bar[s]), (unsigned)(it / STAGES) & 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned base = stage0 + s * STAGE_BYTES;
                    const unsigned long long db = gt_desc(base + A_BYTES);
#pragma unroll
                    for (int a = 0; a < NA; ++a) {
                        const unsigned long long da = gt_desc(base + a * 128 * GT_BK * 2);
#pragma unroll
                        for (int kk = 0; kk < GT_BK / 16; ++kk)      // 16 columns = 32 bytes further inside the swizzle atom
                            gt_mma(acc + a * BN, da + 2ull * kk, db + 2ull * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    gt_commit(gt_smem(&empty_bar[s]));               // the stage is free once these MMAs have read it
                }
                if (ok) gt_commit(gt_smem(&acc_full[buf]));          // all MMAs of the tile done: the accumulator is complete
            }
            if (!ok) { atomicExch(status, 2); abort_s = 1; }
        }
    } else {                                                        // ---------------- epilogue, warps 2..17
        const int quarter = warp & 3;                               // the 32 lanes of tensor memory this warp may read
        const int turn = (warp - 2) >> 2;                           // which of the quarter's four warps: chunks turn, turn + 4, ...
        const int etid = (warp - 2) * 32 + lane;                    // among the epilogue threads
        unsigned char* const box = staging + (warp - 2) * 4096;     // ACCUM: this warp's 4 KB box
        int staged = 0;                                             // ACCUM: boxes this warp has sent
        pdl_wait();
        for (int t = blockIdx.x, lt = 0; t < p.tiles; t += gridDim.x, ++lt) {
            const int buf = lt & 1, m0 = tile_m0(t), n0 = tile_n0(t);
            bool ok = gt_wait(gt_smem(&acc_full[buf]), (unsigned)((lt >> 1) & 1), abort_flag);
            if (EPI == GT_ROPE) ok = gt_epilogue_all(ok);           // (also: the last tile's scatter is over, the staging is free)
            if (!ok) { atomicExch(status, 2); abort_s = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * ACC_COLS);

            gt_epilogue_tile<SWAP, BN, EPI>(p, &map_out, taddr, m0, n0, quarter, turn, lane, staging, box, staged);
            // the accumulator has been read: the tensor core may fill it again
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gt_smem(&acc_empty[buf])) : "memory");
            if (EPI == GT_ROPE) {
                gt_epilogue_sync();                                 // the whole tile is in the staging
                gt_rope_scatter(p, staging, SWAP ? min(BN, p.M - m0) : min(128, p.M - m0), m0, n0, etid);
            }
        }
        if (EPI == GT_ACCUM && !SWAP && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)TMEM_COLS) : "memory");
    }
}


// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// A single SM takes in about 64 bytes a cycle from L2, and a 128 x 256 x 64 step of one CTA needs 48 KB for 512
// cycles of the tensor core: 1.5 times what arrives.  Two CTAs of a cluster therefore share a tile of 256 rows:
// each loads its own 128 rows of A and only HALF of the rows of W (32 KB a step), and one tcgen05.mma with
// cta_group::2, issued by the even CTA, multiplies both halves of A by both halves of W, each CTA's tensor
// memory receiving the 128 rows of its own half of A.  The loads are plain TMA loads of this GPU's memory (no
// multicast); the odd CTA's loads complete on the even CTA's "full" barrier, the even CTA's commits arrive on
// the "empty" and "accumulator full" barriers of both, and the odd CTA's epilogue warps arrive on the even
// CTA's "accumulator empty" barrier.
__device__ __forceinline__ unsigned gt_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned gt_map_to_rank(unsigned local_addr, unsigned rank) {
    unsigned a; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank)); return a;
}
// the barrier may lie in the other CTA of the pair
__device__ __forceinline__ void gt_tma_2d_pair(unsigned dst, const CUtensorMap* map, int x, int y, unsigned cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void gt_mma_pair(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrives on the barrier at this address in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void gt_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void gt_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// BN: rows of W of a pair's tile (256: SWIGLU, 128 gate rows in the even CTA and the 128 up rows that match them in
// the odd one, or 256 plain rows; 128: 64 rows in each CTA).
template <int BN, int EPI>
__global__ void __launch_bounds__(GT_THREADS) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_act,
                                                                       const __grid_constant__ CUtensorMap map_w,
                                                                       const __grid_constant__ CUtensorMap map_out,
                                                                       const GtArgs p, int* status) {
    constexpr unsigned A_BYTES = 128 * GT_BK * 2, B_BYTES = (BN / 2) * GT_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // of one CTA
    constexpr int STAGES = gt_stages(STAGE_BYTES, EPI);
    constexpr int TMEM_COLS = gt_pow2_cols(2 * BN);
    constexpr int OUT_COLS = EPI == GT_SWIGLU ? 128 : BN;
    extern __shared__ __align__(1024) unsigned char gt_mem[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = gt_cluster_rank();                               // 0: issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_blocks = (p.K + GT_BK - 1) / GT_BK;
    const unsigned stage0 = (gt_smem(gt_mem) + 1023u) & ~1023u;
    unsigned char* const staging = gt_mem + (stage0 - gt_smem(gt_mem)) + STAGES * STAGE_BYTES;
    const volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&full_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&empty_bar[s])) : "memory");
        }
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(&acc_full[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gt_smem(&acc_empty[b])), "r"(2 * GT_EPI_WARPS) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                                       // the same warp in both CTAs, the same address
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"((unsigned)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    gt_cluster_sync();                                                     // both CTAs' barriers exist before either signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_base_s;
    pdl_launch_dependents();                                               // (after the allocation: see the kernel above)

    auto tile_m0 = [&](int t) { return (t % p.tiles_m) * 256 + (int)rank * 128; };     // this CTA's rows of A
    auto tile_n0 = [&](int t) { return (t / p.tiles_m) * OUT_COLS; };
    const int my_tiles = pair < p.tiles ? (p.tiles - 1 - pair) / pairs + 1 : 0;

    if (warp == 0) {
        if (lane == 0) {                                            // ---------------- producer (both CTAs)
            const long long total = (long long)my_tiles * k_blocks;
            auto load_w = [&](long long it) {
                const int t = pair + (int)(it / k_blocks) * pairs, kb = (int)(it % k_blocks), s = (int)(it % STAGES);
                const unsigned bar = gt_map_to_rank(gt_smem(&full_bar[s]), 0u), dst = stage0 + s * STAGE_BYTES + A_BYTES;
                const int n0 = tile_n0(t);
                if (rank == 0)                                       // the even CTA's barrier counts the bytes of both
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gt_smem(&full_bar[s])), "r"(2u * STAGE_BYTES) : "memory");
                if (EPI == GT_SWIGLU) gt_tma_2d_pair(dst, &map_w, kb * GT_BK, rank == 0 ? n0 : p.I + n0, bar);
                else gt_tma_2d_pair(dst, &map_w, kb * GT_BK, n0 + (int)rank * (BN / 2), bar);
            };
            auto load_act = [&](long long it) {
                const int t = pair + (int)(it / k_blocks) * pairs, kb = (int)(it % k_blocks), s = (int)(it % STAGES);
                gt_tma_2d_pair(stage0 + s * STAGE_BYTES, &map_act, kb * GT_BK, tile_m0(t), gt_map_to_rank(gt_smem(&full_bar[s]), 0u));
            };
            const long long ahead = total < STAGES ? total : STAGES;
            for (long long it = 0; it < ahead; ++it) load_w(it);
            pdl_wait();
            for (long long it = 0; it < ahead; ++it) load_act(it);
            bool ok = true;
            for (long long it = ahead; it < total; ++it) {
                const int s = (int)(it % STAGES);
                if (!gt_wait(gt_smem(&empty_bar[s]), (unsigned)((it / STAGES) - 1) & 1u, abort_flag)) { ok = false; break; }
                load_w(it);
                load_act(it);
            }
            // before this CTA may end, the commits that the even CTA sends to its "empty" barriers must have arrived
            for (long long it = total > STAGES ? total - STAGES : 0; ok && it < total; ++it)
                if (!gt_wait(gt_smem(&empty_bar[it % STAGES]), (unsigned)(it / STAGES) & 1u, abort_flag)) ok = false;
            if (!ok) { atomicExch(status, 2); abort_s = 1; }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                               // ---------------- MMA issuer (even CTA)
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = BN, M = 256 over the pair
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
            long long it = 0;
            bool ok = true;
            for (int lt = 0; lt < my_tiles && ok; ++lt) {
                const int buf = lt & 1;
                if (!gt_wait(gt_smem(&acc_empty[buf]), (unsigned)((lt >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned acc = tmem + (unsigned)(buf * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    if (!gt_wait(gt_smem(&full_bar[s]), (unsigned)(it / STAGES) & 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned base = stage0 + s * STAGE_BYTES;
                    const unsigned long long da = gt_desc(base), db = gt_desc(base + A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < GT_BK / 16; ++kk)
                        gt_mma_pair(acc, da + 2ull * kk, db + 2ull * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    gt_commit_pair(gt_smem(&empty_bar[s]));
                }
                if (ok) gt_commit_pair(gt_smem(&acc_full[buf]));
            }
            if (!ok) { atomicExch(status, 2); abort_s = 1; }
        }
    } else {                                                        // ---------------- epilogue (both CTAs)
        const int quarter = warp & 3, turn = (warp - 2) >> 2, etid = (warp - 2) * 32 + lane;
        unsigned char* const box = staging + (warp - 2) * 4096;
        int staged = 0;
        pdl_wait();
        for (int lt = 0; lt < my_tiles; ++lt) {
            const int t = pair + lt * pairs, buf = lt & 1, m0 = tile_m0(t), n0 = tile_n0(t);
            bool ok = gt_wait(gt_smem(&acc_full[buf]), (unsigned)((lt >> 1) & 1), abort_flag);
            if (EPI == GT_ROPE) ok = gt_epilogue_all(ok);
            if (!ok) { atomicExch(status, 2); abort_s = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN);
            gt_epilogue_tile<false, BN, EPI>(p, &map_out, taddr, m0, n0, quarter, turn, lane, staging, box, staged);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)                                          // both CTAs' warps count on the even CTA's barrier
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(gt_map_to_rank(gt_smem(&acc_empty[buf]), 0u)) : "memory");
            if (EPI == GT_ROPE) {
                gt_epilogue_sync();
                gt_rope_scatter(p, staging, min(128, p.M - m0), m0, n0, etid);
            }
        }
        if (EPI == GT_ACCUM && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    gt_cluster_sync();                                                     // neither CTA is signalled or written by the other after this
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
static int gt_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows, int box_cols, bool f32) {
    return pe_tensor_map_2d(map, base, rows, cols, box_rows, box_cols, f32);
}

static int gt_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <bool SWAP, int BN, int EPI>
static int gt_launch(const void* A, const void* W, GtArgs& p, int* status, cudaStream_t s) {
    constexpr int NA = (SWAP && EPI == GT_SWIGLU) ? 2 : 1;
    constexpr unsigned STAGE_BYTES = NA * 128 * GT_BK * 2 + BN * GT_BK * 2;
    constexpr int STAGES = gt_stages(STAGE_BYTES, EPI);
    constexpr int OUT_COLS = (!SWAP && EPI == GT_SWIGLU) ? 128 : BN;
    CUtensorMap ma, mw, mo;
    int rc = gt_make_map(&ma, A, p.M, p.K, SWAP ? BN : 128, GT_BK, false);
    if (rc) return rc;
    rc = gt_make_map(&mw, W, p.N, p.K, 128, GT_BK, false);
    if (rc) return rc;
    mo = ma;                                                         // only ACCUM (not swapped) reduces through a map
    if (EPI == GT_ACCUM && !SWAP) {
        rc = gt_make_map(&mo, p.out, p.M, p.N, 32, 32, true);
        if (rc) return rc;
    }
    const int out_n = EPI == GT_SWIGLU ? p.I : p.N;                  // features that tiles are cut from
    p.tiles_m = (p.M + (SWAP ? BN : 128) - 1) / (SWAP ? BN : 128);
    p.tiles = p.tiles_m * ((out_n + (SWAP ? 128 : OUT_COLS) - 1) / (SWAP ? 128 : OUT_COLS));
    const size_t smem = (size_t)STAGES * STAGE_BYTES + gt_staging_bytes(EPI) + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        PE_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<SWAP, BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    const int ctas = p.tiles < gt_sm_count() ? p.tiles : gt_sm_count();
    PE_TRY(pe_launch(gemm_tcgen05_kernel<SWAP, BN, EPI>, dim3(ctas), GT_THREADS, smem, s, ma, mw, mo, p, status));
    return 0;
}

template <int BN, int EPI>
static int gt_launch_pair(const void* A, const void* W, GtArgs& p, int* status, cudaStream_t s) {
    constexpr unsigned STAGE_BYTES = 128 * GT_BK * 2 + (BN / 2) * GT_BK * 2;
    constexpr int STAGES = gt_stages(STAGE_BYTES, EPI);
    constexpr int OUT_COLS = EPI == GT_SWIGLU ? 128 : BN;
    CUtensorMap ma, mw, mo;
    int rc = gt_make_map(&ma, A, p.M, p.K, 128, GT_BK, false);
    if (rc) return rc;
    rc = gt_make_map(&mw, W, p.N, p.K, EPI == GT_SWIGLU ? 128 : BN / 2, GT_BK, false);
    if (rc) return rc;
    mo = ma;
    if (EPI == GT_ACCUM) {
        rc = gt_make_map(&mo, p.out, p.M, p.N, 32, 32, true);
        if (rc) return rc;
    }
    const int out_n = EPI == GT_SWIGLU ? p.I : p.N;
    p.tiles_m = (p.M + 255) / 256;
    p.tiles = p.tiles_m * ((out_n + OUT_COLS - 1) / OUT_COLS);
    const size_t smem = (size_t)STAGES * STAGE_BYTES + gt_staging_bytes(EPI) + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        PE_TRY(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    const int max_pairs = gt_sm_count() / 2, pairs = p.tiles < max_pairs ? p.tiles : max_pairs;
    PE_TRY(pe_launch_cluster(gemm_tcgen05_pair_kernel<BN, EPI>, dim3(2 * pairs), GT_THREADS, smem, s, 2u, ma, mw, mo, p, status));
    return 0;
}

template <int EPI>
static int gt_dispatch(const void* A, const void* W, GtArgs& p, int orientation, int* status, cudaStream_t s) {
    // Left to itself: up to 32 rows swapped (measured at the Qwen2.5-0.5B widths: gate/up at 32 rows 12 us against
    // 20 us; from 64 rows on the orientations are level or "rows" is ahead), CTA pairs from 4096 rows on (3 % ahead
    // at 8192 rows, 3 % behind at 2048).
    const bool swap = orientation == 2 || (orientation == 0 && p.M <= 32);
    if (orientation == 3 || (orientation == 0 && p.M >= 4096)) {     // CTA pairs: 256 rows of A a tile
        if (EPI == GT_SWIGLU || (EPI != GT_ROPE && p.N >= 2048)) return gt_launch_pair<256, EPI>(A, W, p, status, s);
        return gt_launch_pair<128, EPI>(A, W, p, status, s);
    }
    if (!swap) return gt_launch<false, EPI == GT_SWIGLU ? 256 : 128, EPI>(A, W, p, status, s);
    if (p.M <= 32) return gt_launch<true, 32, EPI>(A, W, p, status, s);
    if (p.M <= 64) return gt_launch<true, 64, EPI>(A, W, p, status, s);
    return gt_launch<true, 128, EPI>(A, W, p, status, s);
}

// epilogue 0: out bfloat16 [M, N] = A . W^T + bias;  1: float32 out [M, N] += A . W^T;
//          2: out bfloat16 [M, N / 2] = silu(A . Wg^T) * (A . Wu^T), W = [Wg; Wu]
// orientation 0: chosen by M; 1: rows of A on the accumulator's lanes; 2: rows of W on the lanes (swapped);
//             3: rows of A on the lanes, 256 of them to a pair of CTAs (cta_group::2)
extern "C" int pe_gemm_tcgen05(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                               int M, int N, int K, int orientation, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || N % 8 || epilogue < 0 || epilogue > 2 || orientation < 0 || orientation > 3 || !status) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)out) & 15) return PE_ERR_UNSUPPORTED;
    if (epilogue == 2 && (N % 16 || bias)) return PE_ERR_UNSUPPORTED;
    if (epilogue == 1 && bias) return PE_ERR_UNSUPPORTED;
    GtArgs p = {};
    p.out = out; p.bias = bias; p.bias_dtype = bias_dtype; p.M = M; p.N = N; p.K = K; p.I = N / 2;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == 2) return gt_dispatch<GT_SWIGLU>(A, W, p, orientation, status, s);
    if (epilogue == 0) return gt_dispatch<GT_STORE>(A, W, p, orientation, status, s);
    return gt_dispatch<GT_ACCUM>(A, W, p, orientation, status, s);
}

// q[M, n_q * hd] and the cache pages of keys and values from bfloat16 rows `A`: project with W = [Wq; Wk; Wv],
// add bias, rotate q and k by position (cos_t null: no rotation), write keys and values at (page of the token's
// sequence, position).  Head sizes 16, 32, 64 and 128 (a 128-row tile of W holds whole heads).
extern "C" int pe_gemm_tcgen05_rope(const void* A, const void* W, const void* bias, int bias_dtype, void* q_out, int M, int K,
                                    int n_q, int n_kv, int hd, const float* cos_t, const float* sin_t, const int* tok_pos,
                                    const int* tok_row, void* k_pool, void* v_pool, const int* block_table, int table_stride,
                                    int store, int orientation, int* status, void* stream) {
    if (M <= 0) return 0;
    if (K <= 0 || K % 8 || (hd != 16 && hd != 32 && hd != 64 && hd != 128) || orientation < 0 || orientation > 3 || !status ||
        !tok_pos || (store && (!tok_row || !k_pool || !v_pool || !block_table)))
        return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15)
        return PE_ERR_UNSUPPORTED;
    GtArgs p = {};
    p.out = q_out; p.bias = bias; p.bias_dtype = bias_dtype; p.M = M; p.N = (n_q + 2 * n_kv) * hd; p.K = K;
    p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.cos_t = cos_t; p.sin_t = sin_t; p.tok_pos = tok_pos; p.tok_row = tok_row;
    p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.block_table = block_table; p.table_stride = table_stride; p.store = store;
    return gt_dispatch<GT_ROPE>(A, W, p, orientation, status, (cudaStream_t)stream);
}
