// bfloat16 matrix product on the 5th-generation tensor cores:  D[128, BN] = A[128, K] . B[BN, K]^T
// per CTA, float32 accumulation in tensor memory (TMEM).
//
// Both operands are row-major with K contiguous ("K-major"), which is how activations
// x[tokens, K] and weights w[features, K] lie in memory, so y = x . w^T needs no transpose:
//   * many tokens (prefill):  A = x (128 tokens per tile), B = w (BN features per tile);
//   * few tokens (decode):    A = w (128 features per tile), B = x (all tokens, padded to
//     BN), and the tile in TMEM is y^T, which the epilogue writes transposed.  The product
//     is then a stream of weights through the tensor core at HBM speed; to fill all SMs the
//     K range can be cut (grid.z) into partial sums that a second kernel adds in a fixed
//     order (with the bias).
//
// Inside a CTA: one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) into a
// ring of shared-memory stages; one thread issues tcgen05.mma (4 per stage: K = 64 elements
// = 4 x 16) and commits each stage back to the loader through an mbarrier; four warps read
// the accumulator with tcgen05.ld and write the result.  Every wait on an mbarrier is
// bounded: if it runs out, the CTA records a code in `status`, stops issuing loads, lets
// the copies in flight land, frees its TMEM and returns.
//
// It stands where mischief/lgml calls mul_mat (src/lgml.c:1811-1839: y = x . w^T).
#include <cuda.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_gemm_tcgen05)

namespace {

constexpr int BM = 128;        // rows of A per tile = UMMA M
constexpr int BK = 64;         // K elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr uint32_t SPIN_LIMIT = 4u << 20;
constexpr int STATUS_TIMEOUT = 10;

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  `abort_flag` (shared) short-circuits every later wait once one has run out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(status, STATUS_TIMEOUT);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tcgen05_alloc(uint32_t *dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tcgen05_ld_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the
// 128-byte swizzle in groups of 8 rows (1024 bytes): start address, leading offset 1 (unused
// with a swizzle), stride offset 1024 bytes between row groups, descriptor version 1, layout
// type 2 (SWIZZLE_128B).  Addresses and offsets are in units of 16 bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor of kind::f16: float32 accumulator (bit 4), bfloat16 A and B (bits 7,
// 10), both K-major (bits 15, 16 clear), N / 8 at bit 17, M / 16 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Params {
    int rows_a;       // valid rows of A (tokens, or features when swapped)
    int rows_b;       // valid rows of B
    int k_blocks;     // ceil(K / 64)
    int tiles_a, tiles_b;   // tiles along the rows of A and of B; tile index = tile_b * tiles_a + tile_a
    int kb_per_split; // k blocks per grid.z slice
    int transposed;   // 1: the tile is y^T (A = weights, B = tokens)
    int swiglu;       // 1: feature rows come in (gate, up) pairs; the output is silu(gate) * up, half as wide
    int out_f32;      // output element type
    int ldo;          // row stride of the output in elements
    long long split_stride;   // elements between the partial results of two splits (0: no split)
    void *out;        // y, or the float32 partial results
    const float *bias;        // per feature, or null (only when there is no split)
    int *status;
};

template <int BN>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};

// NACC accumulators in TMEM: 1 when a CTA owns one tile, 2 when it walks several tiles (then
// the epilogue of one tile runs while the products of the next fill the other accumulator).
template <int BN, int STAGES, int NACC>
__global__ void __launch_bounds__(THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                  const __grid_constant__ CUtensorMap map_b, const Params p) {
    pdl_trigger();   // the next kernel may start its own set-up and weight fetch
    extern __shared__ uint8_t smem_raw[];
    // tiles want 1024-byte alignment for the 128-byte swizzle
    uint8_t *tiles = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[NACC], acc_empty[NACC];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    volatile int *abort_flag = &abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.z;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
    const int n_kb = max(kb1 - kb0, 0);
    const int n_tiles = p.tiles_a * p.tiles_b;
    constexpr uint32_t ACC_COLS = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
    constexpr uint32_t TMEM_COLS = ACC_COLS * NACC;
    static_assert(TMEM_COLS <= 512, "the accumulators do not fit tensor memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < NACC; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 128);      // every epilogue thread arrives
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) tcgen05_alloc(&tmem_base_s, TMEM_COLS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // Weights do not depend on the kernels before this one: fetch them for the first
            // stages at once, then wait for the earlier kernels, then fetch the activations.
            const int first = blockIdx.x;
            const int pre = first < n_tiles ? min(n_kb, STAGES) : 0;
            {
                const int tile_a = first % p.tiles_a, tile_b = first / p.tiles_a;
                for (int i = 0; i < pre; ++i) {
                    uint8_t *a_dst = tiles + (size_t)i * Smem<BN>::STAGE_BYTES;
                    mbar_expect_tx(&full_bar[i], Smem<BN>::STAGE_BYTES);
                    if (p.transposed) tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, tile_a * BM, &full_bar[i]);
                    else tma_load_2d(a_dst + Smem<BN>::A_BYTES, &map_b, (kb0 + i) * BK, tile_b * BN, &full_bar[i]);
                }
                pdl_wait();
                for (int i = 0; i < pre; ++i) {
                    uint8_t *a_dst = tiles + (size_t)i * Smem<BN>::STAGE_BYTES;
                    if (p.transposed) tma_load_2d(a_dst + Smem<BN>::A_BYTES, &map_b, (kb0 + i) * BK, tile_b * BN, &full_bar[i]);
                    else tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, tile_a * BM, &full_bar[i]);
                }
            }
            int it = pre, issued = pre;       // k blocks issued so far, over all tiles of this CTA
            bool ok = true;
            for (int tile = first; tile < n_tiles && ok; tile += gridDim.x) {
                const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
                for (int i = (tile == first ? pre : 0); i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1, abort_flag, p.status) || *abort_flag) {
                        ok = false;
                        break;
                    }
                    uint8_t *a_dst = tiles + (size_t)s * Smem<BN>::STAGE_BYTES;
                    uint8_t *b_dst = a_dst + Smem<BN>::A_BYTES;
                    mbar_expect_tx(&full_bar[s], Smem<BN>::STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, tile_a * BM, &full_bar[s]);
                    tma_load_2d(b_dst, &map_b, (kb0 + i) * BK, tile_b * BN, &full_bar[s]);
                    issued = it + 1;
                }
            }
            // On an abort the consumer may never look at the last stages: let their copies land
            // before this CTA's shared memory can be given to another.
            if (*abort_flag) {
                for (int i = max(issued - STAGES, 0); i < issued; ++i) {
                    uint64_t *bar = &full_bar[i % STAGES];
                    const uint32_t parity = (i / STAGES) & 1;
                    for (uint32_t spin = 0; spin < SPIN_LIMIT && !mbar_try_wait(bar, parity); ++spin) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            bool ok = true;
            int it = 0, j = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++j) {
                const int acc = j % NACC;
                // the epilogue must have drained this accumulator (its use NACC tiles ago)
                if (j >= NACC && !mbar_wait(&acc_empty[acc], ((j / NACC) - 1) & 1, abort_flag, p.status)) break;
                tcgen05_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)acc * ACC_COLS;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag, p.status);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * Smem<BN>::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + Smem<BN>::A_BYTES;
                    const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
                        tcgen05_mma_bf16(tmem_acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(&empty_bar[s]);      // the stage is free once these MMAs have read it
                }
                tcgen05_commit(&acc_full[acc]);         // the accumulator is complete once all MMAs are done
            }
        }
    } else {
        // ---------------- epilogue: 4 warps, warp w reads TMEM lanes 32 * (w % 4) .. + 31 ----------------
        pdl_wait();   // nothing is written before the earlier kernels are done (an empty K range gets here at once)
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                   // row of the tile = TMEM lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float *out_f = (float *)p.out + (size_t)split * p.split_stride;
        __nv_bfloat16 *out_h = (__nv_bfloat16 *)p.out;
        const bool f32 = p.out_f32 || p.split_stride != 0;
        int j = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
        const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
        const int acc = j % NACC;
        const uint32_t acc_col = (uint32_t)acc * ACC_COLS;
        const int a_row = tile_a * BM + row;
        const bool ok = mbar_wait(&acc_full[acc], (j / NACC) & 1, abort_flag, p.status);
        tcgen05_fence_after();
        if (ok && n_kb > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tcgen05_ld_16(lane_addr + acc_col + (uint32_t)c0, r);
                tcgen05_wait_ld();
                if (p.transposed) {
                    // tile row = feature (a_row), tile column = token: y[token][feature]
                    const bool row_ok = a_row < p.rows_a;
                    const float b = (p.bias && row_ok) ? p.bias[a_row] : 0.f;
                    if (p.swiglu) {
                        // lanes 2i and 2i+1 hold the gate and the up row of feature a_row / 2
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float v = __uint_as_float(r[j]) + b;
                            const float up = __shfl_xor_sync(0xffffffffu, v, 1);
                            const int token = tile_b * BN + c0 + j;
                            if (row_ok && (lane & 1) == 0 && token < p.rows_b) {
                                const float act = v / (1.0f + expf(-v)) * up;
                                const size_t o = (size_t)token * p.ldo + (a_row >> 1);
                                if (f32) out_f[o] = act;
                                else out_h[o] = __float2bfloat16_rn(act);
                            }
                        }
                    } else if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int token = tile_b * BN + c0 + j;
                            if (token < p.rows_b) {
                                const float v = __uint_as_float(r[j]) + b;
                                if (f32) out_f[(size_t)token * p.ldo + a_row] = v;
                                else out_h[(size_t)token * p.ldo + a_row] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                } else {
                    // tile row = token (a_row), tile column = feature: 16 consecutive features per thread
                    if (a_row < p.rows_a) {
                        const int f0 = tile_b * BN + c0;
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) + ((p.bias && f0 + j < p.rows_b) ? p.bias[f0 + j] : 0.f);
                        if (p.swiglu) {
                            // columns 2j and 2j+1 are the gate and the up of feature (f0 / 2) + j
                            const size_t o = (size_t)a_row * p.ldo + (f0 >> 1);
                            float act[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) act[j] = v[2 * j] / (1.0f + expf(-v[2 * j])) * v[2 * j + 1];
                            if (f0 + 16 <= p.rows_b && (p.ldo & 7) == 0 && !f32) {
                                uint32_t h[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 pr = __floats2bfloat162_rn(act[2 * j], act[2 * j + 1]);
                                    h[j] = *reinterpret_cast<uint32_t *>(&pr);
                                }
                                *reinterpret_cast<uint4 *>(out_h + o) = make_uint4(h[0], h[1], h[2], h[3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (f0 + 2 * j + 1 < p.rows_b) {
                                        if (f32) out_f[o + j] = act[j];
                                        else out_h[o + j] = __float2bfloat16_rn(act[j]);
                                    }
                                }
                            }
                        } else {
                            const size_t o = (size_t)a_row * p.ldo + f0;
                            if (f0 + 16 <= p.rows_b && (p.ldo & 7) == 0) {
                                // whole run in range and 16-byte aligned (f0 is a multiple of 16): vector stores
                                if (f32) {
                                    float4 *dst = reinterpret_cast<float4 *>(out_f + o);
#pragma unroll
                                    for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                                } else {
                                    uint32_t h[8];
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        __nv_bfloat162 pr = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                        h[j] = *reinterpret_cast<uint32_t *>(&pr);
                                    }
                                    uint4 *dst = reinterpret_cast<uint4 *>(out_h + o);
                                    dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
                                    dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    if (f0 + j < p.rows_b) {
                                        if (f32) out_f[o + j] = v[j];
                                        else out_h[o + j] = __float2bfloat16_rn(v[j]);
                                    }
                                }
                            }
                        }
                    }
                }
            }
        } else if (ok && p.split_stride != 0) {
            // a split with no K range still owns its partial result: zeros
            for (int c = 0; c < BN; ++c) {
                const int t = p.transposed ? tile_b * BN + c : a_row, f = p.transposed ? a_row : tile_b * BN + c;
                const int rows_t = p.transposed ? p.rows_b : p.rows_a, rows_f = p.transposed ? p.rows_a : p.rows_b;
                if (t < rows_t && f < rows_f) out_f[(size_t)t * p.ldo + f] = 0.f;
            }
        }
        // this thread has read its part of the accumulator: hand it back to the MMA warp
        tcgen05_fence_before();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, TMEM_COLS);
    }
}

// Sum the partial results of the K splits in split order, add the bias, store.
template <typename TO>
__global__ void splitk_reduce_kernel(const float *__restrict__ part, long long split_stride, int n_splits, const float *__restrict__ bias,
                                     TO *__restrict__ out, int ldo, int rows, int cols) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
        float v = 0.f;
        for (int s = 0; s < n_splits; ++s) v += act_load(part + (size_t)s * split_stride + i);
        if (bias) v += bias[c];
        out[(size_t)r * ldo + c] = from_f32<TO>(v);
    }
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A [rows, K] row-major bfloat16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle,
// zero fill outside the matrix.
int make_map(CUtensorMap *map, const void *base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (enc == nullptr) LGML_FAIL("gemm_tcgen05: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) LGML_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled failed with %d (rows %lld, K %lld, ld %lld, box %d)", (int)r, rows, K, ld, box_rows);
    return 0;
}

template <int BN, int STAGES, int NACC>
int launch(const CUtensorMap &ma, const CUtensorMap &mb, const Params &p, dim3 grid, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * Smem<BN>::STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("gemm_tcgen05: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    lgml_launch(gemm_tcgen05_kernel<BN, STAGES, NACC>, grid, THREADS, smem, stream, ma, mb, p);
    return lgml_launch_status("gemm_tcgen05");
}

}  // namespace

// Floats of scratch that `n_splits` > 1 needs.
LGML_API long long lgml_gemm_tcgen05_scratch_floats(int M, int N, int n_splits) {
    return n_splits > 1 ? (long long)n_splits * M * N : 0;
}

// y[M, N] = x[M, K] . w[N, K]^T (+ bias[N]);  x, w bfloat16 with row strides ldx, ldw (elements);
// y bfloat16 or float32 with row stride ldy.  n_splits > 1 cuts K and needs `scratch`.
// swiglu: the rows of w come in (gate, up) pairs and y[M, N / 2] = silu(gate) * up (no K split then).
// reduce = 0 with n_splits > 1 leaves the partial sums [n_splits, M, N] in scratch for the next
// kernel to add (bias is then not applied).
LGML_API int lgml_gemm_tcgen05(const void *x, const void *w, const float *bias, void *y, int y_f32, int M, int N, int K, int ldx,
                               int ldw, int ldy, int n_splits, float *scratch, int swiglu, int reduce, int *status,
                               cudaStream_t stream) {
    LGML_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
    LGML_REQUIRE(ldx >= K && ldw >= K && ldy >= (swiglu ? N / 2 : N), "gemm_tcgen05: a leading dimension is smaller than its row");
    LGML_REQUIRE(!swiglu || (N % 2 == 0 && n_splits == 1), "gemm_tcgen05: the gated epilogue needs an even N and no K split");
    LGML_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05: row strides (%d, %d) must be multiples of 8 elements (16 bytes) for TMA", ldx, ldw);
    LGML_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned for TMA");
    LGML_REQUIRE(n_splits >= 1 && n_splits <= 64, "gemm_tcgen05: bad split count %d", n_splits);
    LGML_REQUIRE(n_splits == 1 || scratch != nullptr, "gemm_tcgen05: %d K splits need scratch memory", n_splits);
    if (M == 0) return 0;
    const int k_blocks = (K + BK - 1) / BK;
    if (n_splits > k_blocks) n_splits = k_blocks;
    Params p;
    p.k_blocks = k_blocks;
    p.kb_per_split = (k_blocks + n_splits - 1) / n_splits;
    p.out_f32 = y_f32;
    p.ldo = n_splits > 1 ? N : ldy;
    p.split_stride = n_splits > 1 ? (long long)M * N : 0;
    p.out = n_splits > 1 ? (void *)scratch : y;
    p.bias = n_splits > 1 ? nullptr : bias;
    p.status = status;
    p.swiglu = swiglu;
    CUtensorMap ma, mb;
    int rc;
    dim3 grid;
    const bool swap = M <= 256;
    int bn;
    if (swap) {
        bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
        p.transposed = 1;
        p.rows_a = N;
        p.rows_b = M;
        if ((rc = make_map(&ma, w, N, K, ldw, BM))) return rc;
        if ((rc = make_map(&mb, x, M, K, ldx, bn))) return rc;
        p.tiles_a = (N + BM - 1) / BM;
        p.tiles_b = 1;
        grid = dim3(p.tiles_a, 1, n_splits);
    } else {
        bn = 256;
        p.transposed = 0;
        p.rows_a = M;
        p.rows_b = N;
        if ((rc = make_map(&ma, x, M, K, ldx, BM))) return rc;
        if ((rc = make_map(&mb, w, N, K, ldw, bn))) return rc;
        // a persistent grid: one CTA per SM walks the tiles, tile_a fastest, so that the CTAs
        // running at one time share a few column blocks of the weights and all of the activations
        p.tiles_a = (M + BM - 1) / BM;
        p.tiles_b = (N + bn - 1) / bn;
        const int n_tiles = p.tiles_a * p.tiles_b;
        grid = dim3(n_tiles < 148 ? n_tiles : 148, 1, n_splits);
    }
    LGML_REQUIRE(grid.z <= 65535, "gemm_tcgen05: grid too large");
    switch (bn) {
        case 16: rc = launch<16, 6, 1>(ma, mb, p, grid, stream); break;
        case 32: rc = launch<32, 5, 1>(ma, mb, p, grid, stream); break;
        case 64: rc = launch<64, 4, 1>(ma, mb, p, grid, stream); break;
        case 128: rc = launch<128, 6, 1>(ma, mb, p, grid, stream); break;
        default:
            if (swap) rc = launch<256, 4, 1>(ma, mb, p, grid, stream);
            else rc = launch<256, 4, 2>(ma, mb, p, grid, stream);
            break;
    }
    if (rc) return rc;
    if (n_splits > 1 && reduce) {
        const long long total = (long long)M * N;
        const int threads = 256;
        const long long want = (total + threads - 1) / threads;
        const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
        if (y_f32)
            lgml_launch(splitk_reduce_kernel<float>, blocks, threads, 0, stream, scratch, p.split_stride, n_splits, bias, (float *)y, ldy, M, N);
        else
            lgml_launch(splitk_reduce_kernel<__nv_bfloat16>, blocks, threads, 0, stream, scratch, p.split_stride, n_splits, bias, (__nv_bfloat16 *)y, ldy, M, N);
        rc = lgml_launch_status("gemm_tcgen05 split reduce");
    }
    return rc;
}
