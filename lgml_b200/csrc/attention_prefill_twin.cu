// Paged attention for prompts and portions of prompts on the 5th-generation tensor cores
// (tcgen05), two tiles of 128 query rows per CTA, for head sizes 64 and 128.  bfloat16 operands,
// float32 scores, softmax and output.
//
// A CTA takes up to 256 query rows of one KV head: two tiles, each `tt` consecutive new tokens of
// one request times the `hpc` query heads that share the KV head (row = token * hpc + head), and
// walks the request's pages from the first one a query can see to the page of its last token.
// Per page of 64 keys and per tile:
//     S[128, 64]  = Q[128, D] . K[64, D]^T           tcgen05.mma, accumulator in tensor memory
//     softmax: one thread per row reads its 64 scores from tensor memory, keeps the running
//              maximum and sum in float32 (base-2 exponentials) and writes P as bfloat16 back
//              into tensor memory, over the first half of the columns S came from
//     O[128, D] += P[128, 64] . V[64, D]             tcgen05.mma with P read from tensor memory
//                                                    (V is the N-major B operand)
// Each tile has two buffers of scores, and the scores of page j+2 are issued right behind the
// P V product of page j, which read the buffer they go to.  So the scores of the next page are
// there long before a tile's softmax has finished the current one, and the only chain left in
// a tile is softmax after softmax; the products of both tiles run beside it.
// Warps 0-3 are the softmax of tile 0, warps 4-7 of tile 1 (a warp reads the quarter of tensor
// memory's lanes that its index modulo 4 names); one thread of warp 8 issues the products of
// tile 0, one of warp 9 those of tile 1 (a product of 128 rows takes the tensor core at least
// 48 cycles whatever its width, 64 at 128 columns, and the thread that issues it as long: one
// thread for both tiles was the slowest part of a page); one thread of warp 10 issues all TMA
// copies of pages (keys and values in rings of four pages each); warp 11 writes zeros behind
// the last key of the last page of values.
// The running output O is corrected (read, scaled, written back, by the softmax threads) only
// when a row's maximum has grown by more than 8 (base-2 units) since the value its sums are
// relative to; until then the exponentials are taken against that older maximum and stay below
// 2^8, which bfloat16 and the float32 sums hold without loss.
// Products issued by one thread complete in the order of issue.  The kernel leans on that twice:
// the scores of page j+2 of a tile are issued behind the P V product of its page j, so they
// cannot overwrite P before it has been read; and their arrival tells the softmax threads that
// this product is done.
// A wait on an mbarrier names a phase by its parity.  A thread that comes to a barrier two
// phases late would wait for a third, and one that comes a phase early passes at once; every
// barrier here is either waited on phase after phase by its one kind of consumer, which the
// producer cannot overtake, or is used once.
// The CTA takes all 512 columns of the SM's tensor memory.  With its 193 KB of shared memory no
// other kernel of this package that allocates tensor memory (each needs more than 34 KB of
// shared memory) can be resident on the same SM, so the allocation never waits for a CTA that
// itself waits for this kernel.
// Keys are taken from the cache, so this step's own keys are seen at cache precision, as in
// mischief/lgml, which writes the cache before attention reads it
// (lua/lgml/transformer.lua:1838-1839, :2405-2407; formula :1805-1816, scale :1845).
// Waits on mbarriers are bounded.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "page_map.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_prefill_twin)

namespace {
constexpr int PAGE = 64;
constexpr int STAGES = 4;            // pages of keys, and of values, in shared memory
constexpr int ROWS = 128;            // query rows per tile = UMMA M
constexpr int THREADS = 384;         // warps 0-3: softmax of tile 0; 4-7: of tile 1; 8, 9: the products of tile 0, 1; 10: copies; 11: zeros behind the last value
constexpr int ISSUE_WARP = 8, COPY_WARP = 10, HELP_WARP = 11, HELPERS = 32;
constexpr uint32_t SPIN_LIMIT = 1u << 20;   // polls of up to WAIT_HINT_NS each: about a second
constexpr uint32_t WAIT_HINT_NS = 1000;
constexpr uint32_t POLL_SLEEP_NS = 64;
constexpr int STATUS_TIMEOUT = 13;
constexpr uint32_t TMEM_COLS = 512;  // tile t: columns 256 t ..: two buffers of scores (and P) of 64 columns, then the output O
constexpr uint32_t TILE_COLS = 256, O_COL = 128;
constexpr float RESCALE_STEP = 8.f;  // the output is corrected only when a row's maximum has grown by more than this (base-2 units)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void st_shared_16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// shared memory written by threads becomes visible to the tensor core's reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// one 64 x 64 box (columns x0.., all 64 rows of (page, KV head) z) of a cache tensor into swizzled shared memory
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap *map, int x0, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x0), "r"(0), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(WAIT_HINT_NS) : "memory");   // the thread may sleep up to the hint; it wakes when the phase completes
    return ok != 0;
}
// false: the wait ran out (the status word says so) or another thread's did
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    {
        // most phases waited for here are over already: a test that cannot suspend the thread
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
        if (i >= 8) __nanosleep(POLL_SLEEP_NS);
    }
    *abort_flag = 1;
    atomicExch(status, STATUS_TIMEOUT);
    return false;
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
// D[tmem] (+)= A[smem] . B[smem]
__device__ __forceinline__ void tcgen05_mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: A's row i in lane i, two 16-bit elements of K per 32-bit column
__device__ __forceinline__ void tcgen05_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcgen05_ld_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_st_16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tcgen05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// the largest of three in one instruction (NaN operands are passed over, as by fmaxf)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
// two float32 products-and-sums, or sums, in one instruction
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)), "l"(*reinterpret_cast<uint64_t *>(&c)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}
// 2^x in one instruction; 2^(-inf) = 0
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory matrix descriptor, 128-byte swizzle, version 1.  Offsets in units of 16 bytes.
//   K-major operand (rows of 128 bytes, 8-row groups of 1024 bytes): leading 1 (unused), stride 1024.
//   N-major operand (64 elements of N contiguous in 128 bytes, 8 rows of K per 1024 bytes):
//   leading = distance between blocks of 64 along N, stride = distance between groups of 8 along K.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)((leading_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((stride_bytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 operands, A K-major; B K-major or N-major
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_n_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_n_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a swizzled block of 128-byte rows
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

// A wait of a whole warp: its first lane waits (32 lanes polling one mbarrier take turns, some
// 300 cycles even when the phase is long over) and tells the others, so the warp goes on as one
// (loads and stores of tensor memory behind it are instructions of the whole warp).
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, status) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// P = 2^(S scale - m) of one row as bfloat16 over the columns S came from: two a column, key 2 c
// in the low half.  EDGE: keys outside c_lo..c_hi give 0 (whatever their score, NaN included).
// The sums are kept as pairs (even keys, odd keys) in four chains; their order is a function of
// the column only.
template <bool EDGE>
__device__ __forceinline__ void write_p(const uint32_t (&r)[PAGE], uint32_t s_addr, float scale_log2, float neg_m, int c_lo, int c_hi,
                                        float2 (&sum4)[4]) {
    const float2 scale2 = make_float2(scale_log2, scale_log2), neg_m2 = make_float2(neg_m, neg_m);
#pragma unroll
    for (int c0 = 0; c0 < PAGE; c0 += 32) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float2 x = fma2(make_float2(__uint_as_float(r[c0 + i]), __uint_as_float(r[c0 + i + 1])), scale2, neg_m2);
            float2 p = make_float2(ex2(x.x), ex2(x.y));
            if (EDGE) {
                if (c0 + i > c_hi || c0 + i < c_lo) p.x = 0.f;
                if (c0 + i + 1 > c_hi || c0 + i + 1 < c_lo) p.y = 0.f;
            }
            sum4[(i >> 1) & 3] = add2(sum4[(i >> 1) & 3], p);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(p.x, p.y);
            packed[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
        }
        tcgen05_st_16(s_addr + (uint32_t)(c0 >> 1), packed);
    }
}

// D: the head size, 64 or 128 (a page of one head is then whole 64 x 64 boxes of the cache tensor).
// tt: tokens per tile (128 / hpc); a CTA's tile of the list holds up to 2 tt tokens.
template <int D>
__global__ void __launch_bounds__(THREADS, 1) prefill_attention_twin_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16 *__restrict__ q, int ldq,
    const int *__restrict__ positions, const int *__restrict__ tiles, const int *__restrict__ block_table, int max_blocks, int n_pages,
    __nv_bfloat16 *__restrict__ out, int ldo, int H, int Hkv, int hpc, int tt, float scale, int window, int *__restrict__ status) {
    constexpr int KB = D / 64;                              // 64-element blocks along the head dimension
    constexpr uint32_t TILE_BYTES = KB * ROWS * 128;        // the queries of one tile: [KB][128 rows][128 B]
    constexpr uint32_t PAGE_BYTES = KB * PAGE * 128;        // a page of keys [KB][64 keys][128 B] (K-major: row = key), or of values (N-major: 64 dims per row)
    constexpr int CHUNKS_D = D / 8;                         // 16-byte chunks of a row
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *Qs = base, *Ks = Qs + 2 * TILE_BYTES, *Vs = Ks + STAGES * PAGE_BYTES;
    // k_full / v_full: a stage's copy has landed; k_empty / v_empty: the products that read it are
    // done; s_full[t][b]: the scores in buffer b of tile t are there; p_full[t][b]: P is written
    // over them; o_prev[t], o_last[t]: the last but one and the last P V product of tile t are done (a barrier
    // each, used once: a thread that comes late to a barrier of two phases would wait for a third); v_landed: the last page of
    // values is there; v_fixed: zeros stand behind its last key.
    __shared__ uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES], s_full[2][2], p_full[2][2], o_prev[2], o_last[2], v_landed, v_fixed;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    volatile int *abort_flag = &abort_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.y;                  // heads run fastest: the CTAs of one tile start together, tiles in the order given
    const int seq = tiles[tile * 4 + 0], row0 = tiles[tile * 4 + 1], n_tok = tiles[tile * 4 + 2];
    const int group = H / Hkv;
    const int chunks_per_kv = (group + hpc - 1) / hpc;
    const int kvh = blockIdx.x / chunks_per_kv, hchunk = blockIdx.x - kvh * chunks_per_kv;
    const int g0 = hchunk * hpc;                                  // first head of the group this CTA holds
    const int g_count = min(hpc, group - g0);
    const int *table = block_table + (size_t)seq * max_blocks;
    const int pos_first = positions[row0], pos_last = pos_first + n_tok - 1;
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int pg_lo = lo_first / PAGE, pg_hi = pos_last / PAGE;
    const int n_steps = pg_hi - pg_lo + 1;                        // a page a step
    const int n_act = n_tok > tt ? 2 : 1;                         // tiles that hold tokens
    const float scale_log2 = scale * 1.4426950408889634f;
    // The last page's values behind the last key may be anything, NaN included, and 0 x NaN is
    // NaN: they become zeros before the product reads them.  (Keys there give scores that the
    // softmax masks.)
    const int last_rows = pos_last - pg_hi * PAGE + 1;            // rows of the last page that hold keys
    const bool fix_last = last_rows < PAGE;

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], n_act);        // a commit of each tile's issuing thread
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], n_act);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i >> 1][i & 1], 1);
            mbar_init(&p_full[i >> 1][i & 1], ROWS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&o_prev[i], 1);
            mbar_init(&o_last[i], 1);
        }
        mbar_init(&v_landed, 1);
        mbar_init(&v_fixed, HELPERS);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(&tmem_base_s, TMEM_COLS);
    // The positions, tiles and block tables come from the host; everything else this kernel reads
    // (queries, this step's keys and values) is written by the kernels ahead of it.
    pdl_wait();
    // queries: row r of tile t = token (t tt + r / hpc), head g0 + (r % hpc); through L2, they were just written
    // (a thread's loads all go out before its first store: the CTA waits here for one trip to L2, not for eleven)
    constexpr int PER_THREAD = (2 * ROWS * CHUNKS_D + THREADS - 1) / THREADS;
    uint4 v[PER_THREAD];
    uint32_t dst[PER_THREAD];
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int c = tid + i * THREADS;
        const int r2 = c / CHUNKS_D, ch = c - r2 * CHUNKS_D;
        const int t = r2 >> 7, r = r2 & (ROWS - 1);
        const int tok_in = r / hpc, g = r - tok_in * hpc;
        const int tok = t * tt + tok_in;
        // rows without a token or a head get zeros: their scores are then 0 and their sums finite,
        // whatever the pages hold, so a page needs per-element tests only where the mask cuts it
        const bool have = tok_in < tt && tok < n_tok && g < g_count;
        dst[i] = c < 2 * ROWS * CHUNKS_D ? smem_u32(Qs + t * TILE_BYTES + (ch >> 3) * (ROWS * 128)) + swz(r, ch & 7) : 0u;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (dst[i] && have) v[i] = __ldcg(reinterpret_cast<const uint4 *>(q + (size_t)(row0 + tok) * ldq + (size_t)(kvh * group + g0 + g) * D + ch * 8));
    }
    tcgen05_fence_before();
    __syncthreads();                     // the barriers and tensor memory are there; the queries are on their way
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // A page the table does not name is an error of the caller: the status word says so (3), the
    // host raises, and page 0 is read in its place.
    auto page_of = [&](int j) -> int {
        const int page = table[pg_lo + j];
        if (page >= 0 && page < n_pages) return page;
        atomicExch(status, 3);
        return 0;
    };
    auto copy_keys = [&](int j) {
        const int s = j % STAGES, z = page_of(j) * Hkv + kvh;
        mbar_expect_tx(&k_full[s], PAGE_BYTES);
        for (int b = 0; b < KB; ++b) tma_load_box(smem_u32(Ks + s * PAGE_BYTES) + b * (PAGE * 128), &map_k, b * 64, z, &k_full[s]);
    };
    auto copy_values = [&](int j) {
        const int s = j % STAGES, z = page_of(j) * Hkv + kvh;
        mbar_expect_tx(&v_full[s], PAGE_BYTES);
        for (int b = 0; b < KB; ++b) tma_load_box(smem_u32(Vs + s * PAGE_BYTES) + b * (PAGE * 128), &map_v, b * 64, z, &v_full[s]);
    };

    if (warp == COPY_WARP && lane == 0) {
        // in the order the products want them: K(0), K(1), then V(j), K(j + 2)
        copy_keys(0);
        if (n_steps > 1) copy_keys(1);
        for (int j = 0; j + 2 < STAGES && j < n_steps; ++j) {
            copy_values(j);
            if (j + 2 < n_steps) copy_keys(j + 2);
        }
    }
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i)
        if (dst[i]) st_shared_16(dst[i], v[i].x, v[i].y, v[i].z, v[i].w);
    fence_async_smem();
    __syncthreads();

    constexpr uint32_t idesc_qk = make_idesc(ROWS, PAGE, 0);
    constexpr uint32_t idesc_pv = make_idesc(ROWS, D, 1);

    if (warp < 8) {
        // ---- softmax of tile t: one thread per row ----------------------------------------------------
        const int t = warp >> 2;
        const int quarter = warp & 3;                                 // the quarter of tensor memory's lanes this warp may touch
        const int row = quarter * 32 + lane;
        const int my_tok = row / hpc, my_g = row - my_tok * hpc;
        const int n_tok_t = min(max(n_tok - t * tt, 0), tt);
        const bool row_valid = my_tok < n_tok_t && my_g < g_count;
        const int pos_first_t = pos_first + t * tt, pos_last_t = pos_first_t + n_tok_t - 1;
        const int qpos = row_valid ? pos_first_t + my_tok : -1;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)t * TILE_COLS;
        const uint32_t o_addr = lane_addr + O_COL;
        // m_ref: the maximum (base-2 units) that this row's sum l_run and its output in tensor memory
        // are relative to.  It follows the row's running maximum only when that has grown by more
        // than RESCALE_STEP since.
        float m_ref = -INFINITY, l_run = 0.f;
        bool alive = t < n_act;
        for (int j = 0; alive && j < n_steps; ++j) {
            const int key0 = (pg_lo + j) * PAGE, b = j & 1;
            const uint32_t s_addr = lane_addr + (uint32_t)b * PAGE;
            if (!warp_wait(&s_full[t][b], (j >> 1) & 1, abort_flag, status)) {
                alive = false;
                break;
            }
            tcgen05_fence_after();
            // Columns c (keys key0 + c) this row may see: c_lo <= c <= c_hi.  A page that lies wholly
            // inside every row's range takes the path without per-element tests.
            const bool edge = key0 + PAGE - 1 > pos_first_t || (window > 0 && key0 < pos_last_t - window + 1);
            const int c_hi = qpos - key0;                                              // qpos = -1 for a row without a token
            const int c_lo = (window > 0) ? qpos - window + 1 - key0 : -(1 << 30);
            uint32_t r[PAGE];
#pragma unroll
            for (int c0 = 0; c0 < PAGE; c0 += 16) tcgen05_ld_16(s_addr + (uint32_t)c0, *reinterpret_cast<uint32_t(*)[16]>(&r[c0]));
            tcgen05_wait_ld();
            // (four chains each: the order of a maximum or of these float32 partial sums is a
            //  function of the column only, so a row's result does not depend on the batch)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (edge) {
#pragma unroll
                for (int c = 0; c < PAGE; ++c)
                    if (c <= c_hi && c >= c_lo) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(r[c]));
            } else {
#pragma unroll
                for (int c = 0; c < PAGE; c += 8) {
                    mx4[0] = fmax3(mx4[0], __uint_as_float(r[c]), __uint_as_float(r[c + 1]));
                    mx4[1] = fmax3(mx4[1], __uint_as_float(r[c + 2]), __uint_as_float(r[c + 3]));
                    mx4[2] = fmax3(mx4[2], __uint_as_float(r[c + 4]), __uint_as_float(r[c + 5]));
                    mx4[3] = fmax3(mx4[3], __uint_as_float(r[c + 6]), __uint_as_float(r[c + 7]));
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the scale is positive, so the maximum of the raw scores is the maximum of the scaled ones
            const float m_new = mx * scale_log2;
            float corr = 1.f;
            if (m_ref == -INFINITY) {
                m_ref = m_new;                       // nothing summed yet: nothing to correct
            } else if (m_new > m_ref + RESCALE_STEP) {
                corr = ex2(m_ref - m_new);
                m_ref = m_new;
                l_run *= corr;
            }
            if (__any_sync(0xffffffffu, corr != 1.f)) {
                // ---- correct the running output in tensor memory (rare) ----
                // (a correction implies an earlier step: its product into O must be done.  The
                //  scores of step j+1 were issued behind it, so their arrival says so; the last
                //  step has a barrier for it.)
                if (!(j + 1 < n_steps ? warp_wait(&s_full[t][b ^ 1], ((j + 1) >> 1) & 1, abort_flag, status) : warp_wait(&o_prev[t], 0, abort_flag, status))) {
                    alive = false;
                    break;
                }
                tcgen05_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 16) {
                    uint32_t o[16];
                    tcgen05_ld_16(o_addr + (uint32_t)c0, o);
                    tcgen05_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tcgen05_st_16(o_addr + (uint32_t)c0, o);
                }
            }
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;    // keeps (-inf) - (-inf) out of the exponent
            float2 sum4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            if (edge) write_p<true>(r, s_addr, scale_log2, neg_m, c_lo, c_hi, sum4);
            else write_p<false>(r, s_addr, scale_log2, neg_m, c_lo, c_hi, sum4);
            const float2 sum2 = add2(add2(sum4[0], sum4[1]), add2(sum4[2], sum4[3]));
            l_run += sum2.x + sum2.y;
            tcgen05_wait_st();
            tcgen05_fence_before();
            mbar_arrive(&p_full[t][b]);
        }
        // ---- normalise and write this row ----
        if (t < n_act) {
            if (alive && !warp_wait(&o_last[t], 0, abort_flag, status)) alive = false;
            tcgen05_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const bool store = row_valid && alive;
            // (every lane takes part in the loads from tensor memory, which are for whole warps; rows
            //  without a token only skip the stores)
            __nv_bfloat16 *dst = out + (size_t)(row0 + (store ? t * tt + my_tok : 0)) * ldo + (size_t)(kvh * group + g0 + (store ? my_g : 0)) * D;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 16) {
                uint32_t o[16];
                tcgen05_ld_16(o_addr + (uint32_t)c0, o);
                tcgen05_wait_ld();
                if (store) {
#pragma unroll
                    for (int c8 = 0; c8 < 16; c8 += 8) {
                        uint32_t h[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(o[c8 + 2 * i]) * inv, __uint_as_float(o[c8 + 2 * i + 1]) * inv);
                            h[i] = *reinterpret_cast<uint32_t *>(&pr);
                        }
                        *reinterpret_cast<uint4 *>(dst + c0 + c8) = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                }
            }
        }
    } else if ((warp == ISSUE_WARP || warp == ISSUE_WARP + 1) && lane == 0 && warp - ISSUE_WARP < n_act) {
        // ---- the products of tile t: one thread issues them all ----------------------------------------
        // (a thread of its own for each tile: issuing a product and its commits takes the thread
        //  some 50 to 100 cycles each, and 12 products a page and tile are more than one thread
        //  could issue for both tiles in the time the softmax takes)
        const int t = warp - ISSUE_WARP;
        // The descriptors differ from their first one only in the address field (units of 16
        // bytes), so they are made once and advanced by additions.
        const uint64_t desc_q0 = make_desc(smem_u32(Qs + t * TILE_BYTES), 16, 1024), desc_k0 = make_desc(smem_u32(Ks), 16, 1024);
        const uint64_t desc_v0 = make_desc(smem_u32(Vs), PAGE * 128, 1024);
        const uint32_t tile_addr = tmem_base + (uint32_t)t * TILE_COLS;
        auto issue_scores = [&](int j) {          // S_t[j & 1] = Q_t K(j)^T
            const uint64_t dk = desc_k0 + (uint64_t)(((j % STAGES) * PAGE_BYTES) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint64_t da = desc_q0 + (uint64_t)(((ks >> 2) * (ROWS * 128) + (ks & 3) * 32) >> 4);
                const uint64_t db = dk + (uint64_t)(((ks >> 2) * (PAGE * 128) + (ks & 3) * 32) >> 4);
                tcgen05_mma_ss(tile_addr + (uint32_t)(j & 1) * PAGE, da, db, idesc_qk, ks > 0 ? 1u : 0u);
            }
            tcgen05_commit(&s_full[t][j & 1]);
            tcgen05_commit(&k_empty[j % STAGES]);
        };
        auto issue_output = [&](int j) {          // O_t (+)= P_t[j & 1] V(j)
            const uint64_t dv = desc_v0 + (uint64_t)(((j % STAGES) * PAGE_BYTES) >> 4);
#pragma unroll
            for (int k2 = 0; k2 < PAGE / 16; ++k2) {
                // 16 keys further: 8 columns of P; two groups of 8 rows of V (blocks of 64 dims are
                // PAGE * 128 bytes apart: the leading offset of the descriptor)
                tcgen05_mma_ts(tile_addr + O_COL, tile_addr + (uint32_t)(j & 1) * PAGE + (uint32_t)k2 * 8u, dv + (uint64_t)((k2 * 2048) >> 4), idesc_pv,
                               (j > 0 || k2 > 0) ? 1u : 0u);
            }
            if (j + 2 == n_steps) tcgen05_commit(&o_prev[t]);
            if (j + 1 == n_steps) tcgen05_commit(&o_last[t]);
            tcgen05_commit(&v_empty[j % STAGES]);
        };
        // the scores of the first two pages; later ones are issued two pages ahead, behind the
        // P V product that read the buffer they go to
        bool alive = true;
        for (int j = 0; alive && j < 2 && j < n_steps; ++j) {
            if (!mbar_wait(&k_full[j], 0, abort_flag, status)) {
                alive = false;
                break;
            }
            tcgen05_fence_after();
            issue_scores(j);
        }
        for (int j = 0; alive && j < n_steps; ++j) {
            if (!mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1, abort_flag, status)) break;
            if (fix_last && j == n_steps - 1 && !mbar_wait(&v_fixed, 0, abort_flag, status)) break;
            if (!mbar_wait(&p_full[t][j & 1], (j >> 1) & 1, abort_flag, status)) break;
            tcgen05_fence_after();
            issue_output(j);
            if (j + 2 < n_steps) {
                if (!mbar_wait(&k_full[(j + 2) % STAGES], ((j + 2) / STAGES) & 1, abort_flag, status)) break;
                tcgen05_fence_after();
                issue_scores(j + 2);
            }
        }
    } else if (warp == COPY_WARP && lane == 0) {
        // ---- the later copies: a stage is free once the products that read it are done -----------------
        // (V(0 .. STAGES-3) and K(0 .. STAGES-1) went out above)
        bool alive = true;
        for (int j = STAGES - 2; alive && j < n_steps; ++j) {
            if (j >= STAGES && !mbar_wait(&v_empty[j % STAGES], ((j / STAGES) - 1) & 1, abort_flag, status)) break;
            copy_values(j);
            const int j2 = j + 2;
            if (j2 < n_steps) {
                if (!mbar_wait(&k_empty[j2 % STAGES], ((j2 / STAGES) - 1) & 1, abort_flag, status)) break;
                copy_keys(j2);
            }
        }
        // the last page of values is there: the zeros behind its last key may be written
        // (this thread armed that phase of the barrier itself, so it cannot take an older one for it)
        if (fix_last && mbar_wait(&v_full[(n_steps - 1) % STAGES], ((n_steps - 1) / STAGES) & 1, abort_flag, status)) mbar_arrive(&v_landed);
        // no copy of this CTA is in flight when it ends (all have landed long ago unless a wait ran out)
        for (int j = max(n_steps - STAGES, 0); j < n_steps; ++j) {
            mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1, abort_flag, status);
            mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1, abort_flag, status);
        }
    } else if (warp == HELP_WARP && fix_last) {
        // ---- zeros behind the last key of the last page's values: warp 11 ------------------------------
        const int htid = lane, j = n_steps - 1;
        if (warp_wait(&v_landed, 0, abort_flag, status)) {
            const uint32_t dst = smem_u32(Vs + (j % STAGES) * PAGE_BYTES);
            for (int i = htid; i < (PAGE - last_rows) * CHUNKS_D; i += HELPERS) {
                const int zr = last_rows + i / CHUNKS_D, ch = i % CHUNKS_D;
                st_shared_16(dst + (ch >> 3) * (PAGE * 128) + swz(zr, ch & 7), 0u, 0u, 0u, 0u);
            }
            fence_async_smem();
            mbar_arrive(&v_fixed);
        }
    }
    // A CTA of this kernel fills its SM (shared and tensor memory).  It lets the next kernel's CTAs
    // start only now, at its end: released at its start they would pile up behind it, each holding
    // what the ones it waits for still need (see common.cuh).
    pdl_trigger();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------------
template <int D>
int launch(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *tiles, const int *block_table, int max_blocks,
           const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo, int H, int Hkv, int hpc, int tt,
           float scale, int window, int *status, cudaStream_t stream) {
    constexpr int KB = D / 64;
    const size_t smem = 2 * (size_t)KB * ROWS * 128 + 2 * STAGES * (size_t)KB * PAGE * 128 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_twin_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("prefill_attention_twin: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap mk, mv;
    int rc;
    if ((rc = lgml_make_page_map(&mk, k_pages, n_pages, Hkv, D, "prefill_attention_twin"))) return rc;
    if ((rc = lgml_make_page_map(&mv, v_pages, n_pages, Hkv, D, "prefill_attention_twin"))) return rc;
    lgml_launch(prefill_attention_twin_kernel<D>, grid, THREADS, smem, stream, mk, mv, q, ldq, positions, tiles, block_table, max_blocks, n_pages,
                out, ldo, H, Hkv, hpc, tt, scale, window, status);
    return lgml_launch_status("prefill_attention_twin");
}
}  // namespace

// Heads per CTA for a group of `group` query heads per KV head (at most 8) and the tokens of a
// CTA's tile of the list: two tiles of 128 rows / heads per CTA.
LGML_API void lgml_prefill_attention_twin_shape(int group, int *heads_per_cta, int *tile_tokens) {
    const int hpc = group < 8 ? group : 8;
    *heads_per_cta = hpc;
    *tile_tokens = 2 * (ROWS / hpc);
}

// 1 if the kernel takes this head size (its pages must be whole 64 x 64 boxes for TMA).
LGML_API int lgml_prefill_attention_twin_takes(int D) { return D == 64 || D == 128; }

LGML_API int lgml_prefill_attention_twin(const void *q, int ldq, const int *positions, const int *tiles, int n_tiles, const int *block_table,
                                         int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, void *out,
                                         int ldo, int H, int Hkv, int D, float scale, int window, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tiles >= 0 && H > 0 && Hkv > 0 && max_blocks > 0 && n_pages > 0, "prefill_attention_twin: bad sizes");
    LGML_REQUIRE(page_size == PAGE, "prefill_attention_twin: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0, "prefill_attention_twin: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D == 64 || D == 128, "prefill_attention_twin: head_dim %d (this kernel takes 64 and 128)", D);
    LGML_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0,
                 "prefill_attention_twin: q and out must be 16-byte aligned with row strides that are multiples of 8");
    LGML_REQUIRE(((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0, "prefill_attention_twin: the cache must be 16-byte aligned");
    if (n_tiles == 0) return 0;
    const int group = H / Hkv;
    int hpc, tile_tokens;
    lgml_prefill_attention_twin_shape(group, &hpc, &tile_tokens);
    const int chunks = (group + hpc - 1) / hpc;
    LGML_REQUIRE((long long)Hkv * chunks <= 65535, "prefill_attention_twin: too many heads");
    LGML_REQUIRE(n_tiles <= 65535, "prefill_attention_twin: %d tiles in one launch (at most 65535)", n_tiles);
    dim3 grid(Hkv * chunks, n_tiles);
    const __nv_bfloat16 *qq = (const __nv_bfloat16 *)q, *kk = (const __nv_bfloat16 *)k_pages, *vv = (const __nv_bfloat16 *)v_pages;
    __nv_bfloat16 *oo = (__nv_bfloat16 *)out;
    if (D == 64)
        return launch<64>(grid, qq, ldq, positions, tiles, block_table, max_blocks, kk, vv, n_pages, oo, ldo, H, Hkv, hpc, tile_tokens / 2, scale, window, status, stream);
    return launch<128>(grid, qq, ldq, positions, tiles, block_table, max_blocks, kk, vv, n_pages, oo, ldo, H, Hkv, hpc, tile_tokens / 2, scale, window, status, stream);
}
