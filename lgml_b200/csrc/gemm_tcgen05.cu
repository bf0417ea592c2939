// bfloat16 matrix product on the 5th-generation tensor cores:  D[128, BN] = A[128, K] . B[BN, K]^T
// per CTA, float32 accumulation in tensor memory (TMEM).
//
// Both operands are row-major with K contiguous ("K-major"), which is how activations
// x[tokens, K] and weights w[features, K] lie in memory, so y = x . w^T needs no transpose:
//   * many tokens (prefill):  A = x (128 tokens per tile), B = w (BN features per tile); from
//     512 tokens on, two CTAs share a 256 x 256 tile (tcgen05.mma.cta_group::2, below);
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

// silu(gate) * up for the gated epilogue, whose result is rounded to bfloat16: the fast exponential
// and division (a few units in the last place of float32, far below that rounding) instead of the
// library's, which cost the epilogue of a 64-token tile more than its loads from tensor memory.
__device__ __forceinline__ float silu_mul_fast(float gate, float up) { return __fdividef(gate, 1.0f + __expf(-gate)) * up; }

// One thread's 16 consecutive features f0 .. f0 + 15 of token row a_row (tile row = token,
// tile column = feature): bias, the gated activation if asked for, and the store.
__device__ __forceinline__ void store_run(const Params &p, int a_row, int f0, const uint32_t (&r)[16], float *out_f, __nv_bfloat16 *out_h,
                                          bool f32) {
    if (a_row < p.rows_a) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) + ((p.bias && f0 + j < p.rows_b) ? p.bias[f0 + j] : 0.f);
        if (p.swiglu) {
            // columns 2j and 2j+1 are the gate and the up of feature (f0 / 2) + j
            const size_t o = (size_t)a_row * p.ldo + (f0 >> 1);
            float act[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) act[j] = silu_mul_fast(v[2 * j], v[2 * j + 1]);
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

// The same for a tile whose rows are features and whose columns are tokens (the weights were the
// tile's rows): one thread's feature a_row for the 16 tokens token0 .. token0 + 15, y[token][feature].
// With the gated activation lanes 2i and 2i+1 hold the gate and the up row of feature a_row / 2.
__device__ __forceinline__ void store_run_transposed(const Params &p, int a_row, int token0, const uint32_t (&r)[16], int lane, float *out_f,
                                                     __nv_bfloat16 *out_h, bool f32) {
    const bool row_ok = a_row < p.rows_a;
    const float b = (p.bias && row_ok) ? p.bias[a_row] : 0.f;
    if (p.swiglu) {
        // Lanes 2i and 2i+1 hold the gate and the up row of one feature.  Of every two tokens the
        // even lane finishes the first and the odd lane the second: one exchange for two tokens
        // (the even lane gives its gate of the second token, the odd lane its up of the first),
        // and both lanes compute and store.
        const bool even = (lane & 1) == 0;
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float v0 = __uint_as_float(r[j]) + b, v1 = __uint_as_float(r[j + 1]) + b;
            const float got = __shfl_xor_sync(0xffffffffu, even ? v1 : v0, 1);
            const int token = token0 + j + (even ? 0 : 1);
            if (row_ok && token < p.rows_b) {
                const float act = even ? silu_mul_fast(v0, got) : silu_mul_fast(got, v1);
                const size_t o = (size_t)token * p.ldo + (a_row >> 1);
                if (f32) out_f[o] = act;
                else out_h[o] = __float2bfloat16_rn(act);
            }
        }
    } else if (row_ok) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int token = token0 + j;
            if (token < p.rows_b) {
                const float v = __uint_as_float(r[j]) + b;
                if (f32) out_f[(size_t)token * p.ldo + a_row] = v;
                else out_h[(size_t)token * p.ldo + a_row] = __float2bfloat16_rn(v);
            }
        }
    }
}

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
    // Few tokens (two CTAs an SM): the next kernel may start its own set-up and weight fetch at once.
    // A CTA that fills its SM triggers at its end instead (see common.cuh).
    constexpr bool EARLY_TRIGGER = BN <= 64;
    if (EARLY_TRIGGER) pdl_trigger();
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
                    store_run_transposed(p, a_row, tile_b * BN + c0, r, lane, out_f, out_h, f32);
                } else {
                    store_run(p, a_row, tile_b * BN + c0, r, out_f, out_h, f32);
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
    if (!EARLY_TRIGGER) pdl_trigger();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, TMEM_COLS);
    }
}


// ---- two CTAs on one tile -------------------------------------------------------------------------
// For many tokens: a cluster of two CTAs (two SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA holds half of the rows of A (128 tokens) and half of the
// rows of B (128 features), so per 64 elements of K it stages 32 KB instead of the 48 KB a lone
// CTA moves for a 128 x 256 tile; shared-memory traffic per flop, which bounds the single-CTA
// kernel, drops by a third.  A stage holds 128 elements of K (64 KB, three stages): the cost of
// a stage's barriers and commits, not their latency, was what held the pairs back with 64.
// The even CTA of the pair (the leader) issues the products; the accumulator of each CTA's 128
// rows lands in that CTA's tensor memory, and each CTA's epilogue warps store their own rows.
// Measured at 2,048 tokens against the single-CTA kernel: 1.38 against 1.26 PFLOP/s (N 6144,
// K 4096), 1.50 against 1.37 (N 28672 with the gated epilogue), 1.44 against 1.30 (K 14336).
//   full_bar[s]   (leader)    both CTAs' TMA copies of stage s have landed (the other CTA's copies
//                             count their bytes on the leader's barrier)
//   empty_bar[s]  (each CTA)  the products have read stage s (tcgen05.commit, multicast to both)
//   acc_full[a]   (each CTA)  accumulator a is complete (commit, multicast to both)
//   acc_empty[a]  (leader)    both CTAs' epilogue threads have read accumulator a (256 arrivals)
// PBN: columns of the pair's tile (256, or 192 or 128 when 256 would leave pairs idle); each CTA
// loads PBN / 2 rows of B.
constexpr int PAIR_KSUB = 2;               // 64-element k blocks per stage
constexpr int PAIR_A_BYTES = BM * BK * 2;                                          // one k block of A
__host__ __device__ constexpr int pair_stage_bytes(int pbn) { return PAIR_KSUB * (PAIR_A_BYTES + (pbn / 2) * BK * 2); }   // [A k0][A k1]..[B k0][B k1]..
constexpr int PAIR_ACC_COLS = 256;          // tensor-memory columns between the two accumulators

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint64_t *bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(smem_u32(bar)), "r"(rank) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(status, STATUS_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tcgen05_alloc_pair(uint32_t *dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the products issued so far are done
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t *bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// A TMA copy into this CTA's shared memory whose bytes are counted on a barrier of the pair's
// leader (`bar_cluster`: a shared::cluster address from mapa).
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ uint32_t mapa_u32(const void *p, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(p)), "r"(rank));
    return ra;
}

template <int PAIR_BN, int STAGES, int PAIR_NACC, bool YT>      // YT: the tile is y^T (the weights are its rows)
__global__ void __launch_bounds__(THREADS, 1) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *tiles = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[PAIR_NACC], acc_empty[PAIR_NACC];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    volatile int *abort_flag = &abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0: the leader, which issues the products
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_kb = (p.k_blocks + PAIR_KSUB - 1) / PAIR_KSUB;      // stages along all of K
    const int n_tiles = p.tiles_a * p.tiles_b;          // tiles of 256 x 256
    // A pair's work is a list of units: unit u is tile u % n_tiles over K range u / n_tiles (stages
    // [range * kb_per_split, ...)); one range unless the tiles alone would leave pairs idle.
    const int per_range = p.kb_per_split;               // stages per K range
    const int n_ranges = (n_kb + per_range - 1) / per_range;
    const int n_units = n_tiles * n_ranges;
    constexpr int PAIR_HALF = PAIR_BN / 2, PAIR_B_BYTES = PAIR_HALF * BK * 2, PAIR_STAGE_BYTES = pair_stage_bytes(PAIR_BN);
    constexpr uint32_t ACC_COLS = PAIR_ACC_COLS;
    constexpr uint32_t TMEM_COLS = ACC_COLS * PAIR_NACC;
    static_assert(PAIR_BN % 32 == 0 && PAIR_BN <= 256 && PAIR_STAGE_BYTES % 1024 == 0, "tile width");

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < PAIR_NACC; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 256);      // the epilogue threads of both CTAs arrive
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) tcgen05_alloc_pair(&tmem_base_s, TMEM_COLS);
    tcgen05_fence_before();
    cluster_sync_all();             // both CTAs' barriers exist before anything arrives on them from the other side
    tcgen05_fence_after();
    // The products name one accumulator address for both CTAs: the leader's.  (Both CTAs take
    // part in one allocation and get the same address; reading the leader's keeps this right
    // even if they did not.)
    uint32_t tmem_base;
    {
        uint32_t ra;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(&tmem_base_s)), "r"(0u));
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(tmem_base) : "r"(ra) : "memory");
    }

    if (warp == 0) {
        // ---------------- TMA producer (each CTA loads its halves) ----------------
        if (lane == 0) {
            // This pair's work is a list of (tile, k block) items; item q goes to stage q % STAGES.
            // Weights do not depend on the kernels before this one: those of the first STAGES items
            // go out at once, then the wait for the earlier kernels, then the activations.  The bytes
            // of both CTAs' copies of a stage are counted on the leader's barrier of that stage,
            // which the leader arms for both.
            uint32_t bar_of[STAGES];
#pragma unroll
            for (int s = 0; s < STAGES; ++s) bar_of[s] = mapa_u32(&full_bar[s], 0);
            int q = 0;
            int first_row[STAGES], first_kb[STAGES];     // where the activations of the first STAGES items lie
            bool waited = false, ok = true;
            // the weights are B (tokens are the tile's rows), or A when the tile is y^T
            constexpr bool w_is_a = YT;
            for (int unit = pair; unit < n_units && ok; unit += n_pairs) {
                const int tile = unit % n_tiles, range = unit / n_tiles;
                const int row_a = (tile % p.tiles_a) * 2 * BM + (int)rank * BM;
                const int row_b = (tile / p.tiles_a) * PAIR_BN + (int)rank * PAIR_HALF;
                const int kb_end = min(n_kb, (range + 1) * per_range);
                for (int kb = range * per_range; kb < kb_end; ++kb, ++q) {
                    const int s = q % STAGES;
                    if (q < STAGES) {
                        first_row[q] = w_is_a ? row_b : row_a;
                        first_kb[q] = kb;
                    }
                    if (q == STAGES && !waited) {
                        // the activations of the first STAGES items, whose weights are under way
                        pdl_wait();
                        waited = true;
#pragma unroll
                        for (int q2 = 0; q2 < STAGES; ++q2) {
#pragma unroll
                            for (int u = 0; u < PAIR_KSUB; ++u) {
                                uint8_t *st = tiles + (size_t)q2 * PAIR_STAGE_BYTES;
                                if (w_is_a) tma_load_2d_pair(st + PAIR_KSUB * PAIR_A_BYTES + u * PAIR_B_BYTES, &map_b, (first_kb[q2] * PAIR_KSUB + u) * BK, first_row[q2], bar_of[q2]);
                                else tma_load_2d_pair(st + u * PAIR_A_BYTES, &map_a, (first_kb[q2] * PAIR_KSUB + u) * BK, first_row[q2], bar_of[q2]);
                            }
                        }
                    }
                    if (q >= STAGES && (!mbar_wait(&empty_bar[s], ((q / STAGES) - 1) & 1, abort_flag, p.status) || *abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t *a_dst = tiles + (size_t)s * PAIR_STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * PAIR_STAGE_BYTES);
#pragma unroll
                    for (int u = 0; u < PAIR_KSUB; ++u) {
                        if (waited || w_is_a) tma_load_2d_pair(a_dst + u * PAIR_A_BYTES, &map_a, (kb * PAIR_KSUB + u) * BK, row_a, bar_of[s]);
                        if (waited || !w_is_a) tma_load_2d_pair(a_dst + PAIR_KSUB * PAIR_A_BYTES + u * PAIR_B_BYTES, &map_b, (kb * PAIR_KSUB + u) * BK, row_b, bar_of[s]);
                    }
                }
            }
            if (!waited) {
                // fewer items than stages: their activations are still to come
                pdl_wait();
#pragma unroll
                for (int q2 = 0; q2 < STAGES; ++q2) {
                    if (q2 < q) {
#pragma unroll
                        for (int u = 0; u < PAIR_KSUB; ++u) {
                            uint8_t *st = tiles + (size_t)q2 * PAIR_STAGE_BYTES;
                            if (w_is_a) tma_load_2d_pair(st + PAIR_KSUB * PAIR_A_BYTES + u * PAIR_B_BYTES, &map_b, (first_kb[q2] * PAIR_KSUB + u) * BK, first_row[q2], bar_of[q2]);
                            else tma_load_2d_pair(st + u * PAIR_A_BYTES, &map_a, (first_kb[q2] * PAIR_KSUB + u) * BK, first_row[q2], bar_of[q2]);
                        }
                    }
                }
            }
            // (On an abort copies may still be in flight; the cluster barrier at the end of the
            // kernel keeps both CTAs, and so their shared memory, until the leader has gone through
            // its bounded waits.)
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---------------- MMA issuer (leader) ----------------
            constexpr uint32_t idesc = make_idesc(2 * BM, PAIR_BN);
            bool ok = true;
            int it = 0, j = 0;
            for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++j) {
                const int acc = j % PAIR_NACC;
                if (j >= PAIR_NACC && !mbar_wait_cluster(&acc_empty[acc], ((j / PAIR_NACC) - 1) & 1, abort_flag, p.status)) break;
                tcgen05_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)acc * ACC_COLS;
                const int range = unit / n_tiles;
                const int stages_here = min(n_kb, (range + 1) * per_range) - range * per_range;
                for (int i = 0; i < stages_here; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag, p.status);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * PAIR_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + PAIR_KSUB * PAIR_A_BYTES;
#pragma unroll
                    for (int u = 0; u < PAIR_KSUB; ++u) {
                        const uint64_t da = make_smem_desc(a_addr + u * PAIR_A_BYTES), db = make_smem_desc(b_addr + u * PAIR_B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            tcgen05_mma_bf16_pair(tmem_acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > 0 || u > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit_pair(&empty_bar[s]);
                }
                tcgen05_commit_pair(&acc_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue: 4 warps per CTA, each CTA its own 128 rows ----------------
        pdl_wait();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        __nv_bfloat16 *out_h = (__nv_bfloat16 *)p.out;
        const bool f32 = p.out_f32 != 0 || p.split_stride != 0;      // the partial sums of K ranges are float32
        int j = 0;
        for (int unit = pair; unit < n_units; unit += n_pairs, ++j) {
            const int tile = unit % n_tiles;
            float *out_f = (float *)p.out + (size_t)(unit / n_tiles) * p.split_stride;
            const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
            const int acc = j % PAIR_NACC;
            const uint32_t acc_col = (uint32_t)acc * ACC_COLS;
            const int a_row = tile_a * 2 * BM + (int)rank * BM + row;
            const bool ok = mbar_wait(&acc_full[acc], (j / PAIR_NACC) & 1, abort_flag, p.status);
            tcgen05_fence_after();
            if (ok) {
#pragma unroll 1
                for (int c0 = 0; c0 < PAIR_BN; c0 += 16) {
                    if (YT && tile_b * PAIR_BN + c0 >= p.rows_b) break;      // columns past the last token
                    uint32_t r[16];
                    tcgen05_ld_16(lane_addr + acc_col + (uint32_t)c0, r);
                    tcgen05_wait_ld();
                    if constexpr (YT) store_run_transposed(p, a_row, tile_b * PAIR_BN + c0, r, lane, out_f, out_h, f32);
                    else store_run(p, a_row, tile_b * PAIR_BN + c0, r, out_f, out_h, f32);
                }
            }
            // this thread has read its part of the accumulator: tell the leader's MMA warp
            tcgen05_fence_before();
            if (rank == 0) asm volatile("mbarrier.arrive.release.cluster.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
            else mbar_arrive_remote(&acc_empty[acc], 0);
        }
    }
    pdl_trigger();      // at the end: a pair fills two SMs, the next kernel's CTAs start when it is done (see common.cuh)
    // nobody leaves, and no tensor memory is given back, while the other CTA may still arrive on
    // this one's barriers or the leader's products may still use this one's memory
    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc_pair(tmem_base, TMEM_COLS);
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

// How many pairs of CTAs the device runs at one time (pairs need both SMs of a TPC, and not
// every TPC of a part has two): the persistent grid is this many pairs, never more, or the
// rest would wait for a second round.  0 if the query fails.
template <int PBN, int STAGES, int NACC, bool YT>
int pairs_at_once(size_t smem) {
    static int n = -1;
    if (n < 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 74);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<PBN, STAGES, NACC, YT>, &cfg);
        n = (e == cudaSuccess && clusters > 0) ? clusters : 0;
        if (e != cudaSuccess) cudaGetLastError();
    }
    return n;
}

template <int PBN, int STAGES, int NACC, bool YT>
int launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, const Params &p, int n_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * pair_stage_bytes(PBN) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<PBN, STAGES, NACC, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("gemm_tcgen05: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int at_once = pairs_at_once<PBN, STAGES, NACC, YT>(smem);
    if (at_once <= 0) LGML_FAIL("gemm_tcgen05: the device runs no pair of CTAs of this kernel");
    const int n_pairs = n_tiles < at_once ? n_tiles : at_once;
    cudaError_t e = lgml_launch_cluster(gemm_pair_kernel<PBN, STAGES, NACC, YT>, dim3(2 * n_pairs), dim3(THREADS), smem, stream, 2, ma, mb, p);
    if (e != cudaSuccess) LGML_FAIL("gemm_tcgen05: launch of CTA pairs failed: %s", cudaGetErrorString(e));
    return lgml_launch_status("gemm_tcgen05 pairs");
}

// From this many tokens on a product runs on pairs of CTAs.  (Up to 64 the weights are the tile's
// rows and the tokens its columns, two CTAs an SM: gate/up product alone at 64 tokens 45 us.  Beyond,
// that shape reads the activations again for every 128 rows of weights and needs a second round
// for a third of its tiles: 71 us at 96 tokens, 112 at 256, where pairs take 60 to 63.)
constexpr int PAIR_MIN_TOKENS = 65;
// Up to this many tokens the pairs' tiles are y^T as well (256 rows of weights, the tokens as the
// tile's 128 columns): with the tokens as rows half of a 256-row tile would be padding, and the
// products of a tile, which bound a pair, twice what they have to be.
constexpr int PAIR_SWAP_TOKENS = 128;

// How a product of M tokens runs on pairs: y^T or not, the tile's width, and how many tiles.
struct PairPlan {
    bool swapped;
    int pbn, tiles_a, tiles_b;
};
int pair_tile_width(int M, int N);
inline PairPlan pair_plan(int M, int N) {
    PairPlan pl;
    pl.swapped = M <= PAIR_SWAP_TOKENS;
    if (pl.swapped) {
        pl.pbn = 128;
        pl.tiles_a = (N + 2 * BM - 1) / (2 * BM);
        pl.tiles_b = (M + pl.pbn - 1) / pl.pbn;
    } else {
        pl.pbn = pair_tile_width(M, N);
        pl.tiles_a = (M + 2 * BM - 1) / (2 * BM);
        pl.tiles_b = (N + pl.pbn - 1) / pl.pbn;
    }
    return pl;
}

// The width of the pairs' tiles for an M x N product: 256 unless a narrower tile fills the 74
// pairs better (few tokens: 512 x 4096 is 32 tiles of 256 columns but 64 of 128).  The cost of a
// tile is taken as its width plus a fixed part; a narrower tile must win by more than 5 %.
int pair_tile_width(int M, int N) {
    const int widths[3] = {256, 192, 128};
    int best = 256;
    double best_cost = 0;
    for (int i = 0; i < 3; ++i) {
        const int w = widths[i];
        const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + w - 1) / w);
        const double cost = (double)((tiles + 73) / 74) * (w + 40);
        if (i == 0 || cost < 0.95 * best_cost) {
            best = w;
            best_cost = cost;
        }
    }
    return best;
}

// LGML_GEMM_PAIR=0: never use CTA pairs (every product of many tokens on single CTAs).
bool pairs_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("LGML_GEMM_PAIR");
        on = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

}  // namespace

// K ranges that a product of M tokens should be cut into when it runs on pairs of CTAs (0: it does
// not run on pairs): as many as fill the 74 pairs once over, each of at least four stages of 128
// elements, at most eight (every range writes, and the next kernel reads, M x N float32 partial sums).
LGML_API int lgml_gemm_tcgen05_pair_ranges(int M, int N, int K) {
    if (M < PAIR_MIN_TOKENS || !pairs_enabled() || N <= 0 || K <= 0) return 0;
    const PairPlan pl = pair_plan(M, N);
    const long long tiles = (long long)pl.tiles_a * pl.tiles_b;
    const int stages = ((K + BK - 1) / BK + PAIR_KSUB - 1) / PAIR_KSUB;
    long long want = 74 / (tiles > 0 ? tiles : 1);
    if (want > stages / 4) want = stages / 4;
    if (want > 8) want = 8;
    if (want < 2) return 1;
    const int per = (int)((stages + want - 1) / want);
    return (stages + per - 1) / per;
}

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
    const bool pair_path = M >= PAIR_MIN_TOKENS && pairs_enabled();
    const bool swap = M <= 256 && !pair_path;
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
    } else if (pair_path) {
        // more than 64 tokens: pairs of CTAs on 256 x 256 tiles, tile_a fastest; K in n_splits ranges of
        // whole stages (128 elements) where the tiles alone would leave pairs idle
        const int stages = (k_blocks + PAIR_KSUB - 1) / PAIR_KSUB;
        p.kb_per_split = (stages + n_splits - 1) / n_splits;
        LGML_REQUIRE((n_splits - 1) * p.kb_per_split < stages, "gemm_tcgen05: %d K ranges of %d stages leave one empty (K = %d)", n_splits,
                     p.kb_per_split, K);
        const PairPlan pl = pair_plan(M, N);
        const int pbn = pl.pbn;
        if (pl.swapped) {
            // the tile is y^T: its rows are features (each CTA of a pair 128 of them), its columns the tokens
            p.transposed = 1;
            p.rows_a = N;
            p.rows_b = M;
            if ((rc = make_map(&ma, w, N, K, ldw, BM))) return rc;
            if ((rc = make_map(&mb, x, M, K, ldx, pbn / 2))) return rc;
        } else {
            p.transposed = 0;
            p.rows_a = M;
            p.rows_b = N;
            if ((rc = make_map(&ma, x, M, K, ldx, BM))) return rc;
            if ((rc = make_map(&mb, w, N, K, ldw, pbn / 2))) return rc;
        }
        p.tiles_a = pl.tiles_a;
        p.tiles_b = pl.tiles_b;
        const int n_tiles = p.tiles_a * p.tiles_b;
        const int n_units = n_tiles * n_splits;
        if (pl.swapped) rc = launch_pair<128, 4, 2, true>(ma, mb, p, n_units, stream);
        else if (pbn == 128) rc = launch_pair<128, 4, 2, false>(ma, mb, p, n_units, stream);
        else if (pbn == 192) rc = launch_pair<192, 4, 2, false>(ma, mb, p, n_units, stream);
        else rc = launch_pair<256, 3, 2, false>(ma, mb, p, n_units, stream);
        bn = 0;      // launched
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
    LGML_REQUIRE(bn == 0 || grid.z <= 65535, "gemm_tcgen05: grid too large");
    switch (bn) {
        case 0: break;
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
