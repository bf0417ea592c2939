// Paged attention for prompts and portions of prompts on the 5th-generation tensor cores
// (tcgen05), bfloat16 operands, float32 scores, softmax and output.
//
// A CTA takes 128 query rows of one KV head: `tt` consecutive new tokens of one request times
// the `hpc` query heads that share the KV head (row = token * hpc + head), and walks the
// request's pages from the first one a query can see to the page of its last token.  Per page
// of 64 keys:
//     S[128, 64]  = Q[128, D] . K_page[64, D]^T      tcgen05.mma, accumulator in tensor memory
//     softmax: one thread per row reads its 64 scores from TMEM, keeps the running maximum and
//              sum in float32 (base-2 exponentials), writes P as bfloat16 to shared memory
//     O[128, D] += P[128, 64] . V_page[64, D]        tcgen05.mma, accumulated in tensor memory (V is the
//                                                    N-major B operand)
// The running output O is corrected (read, scaled, written back) only when a row's maximum has
// grown by more than 8 (base-2 units) since the value its sums are relative to; until then the
// exponentials are taken against that older maximum and stay below 2^8, which bfloat16 and the
// float32 sums hold without loss.  So a page costs one read of its scores from tensor memory
// and nothing for the output; O is read once, at the end, and divided by the row's sum.
// Q, K, V and P sit in shared memory in the 128-byte-swizzled layout the tensor core reads.
// Warps 0-3 do the softmax (one thread per row).  For head sizes that are multiples of 64 the
// pages come by TMA (a page of one head is then whole 64 x 64 boxes of the cache tensor): one
// thread of warp 5 issues the copies (K two pages ahead, V one), one thread of warp 4 the
// products, the scores of page i+1 ahead of the P V product of page i, into a second S
// buffer.  For other head sizes warps 4-7 copy the pages with cp.async and their first thread
// issues the products.  Warps 4-7 also do the rare corrections of O, and all 8 warps write
// the output.  Two CTAs share an SM, so that one's products overlap the other's softmax.  CTAs
// are started with the longest tiles first (the caller orders them).  Keys are taken from the
// cache, so this step's own keys are seen at cache precision, as in mischief/lgml, which writes
// the cache before attention reads it (lua/lgml/transformer.lua:1838-1839, :2405-2407; formula
// :1805-1816, scale :1845).  Waits on mbarriers are bounded.
// A page takes this kernel about 3,400 cycles per CTA, of which the tensor core works 560: what
// bounds it is the chain scores -> softmax (1,000 cycles) -> barrier -> issue of 12 small
// products by one thread (1,200 cycles: about 80 a product, whatever its size) -> scores.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "page_map.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_prefill_tc)

namespace {
constexpr int PAGE = 64;
constexpr int ROWS = 128;            // query rows per CTA = UMMA M
constexpr int THREADS = 256;
constexpr uint32_t SPIN_LIMIT = 1u << 20;   // polls of up to WAIT_HINT_NS each: about a second
constexpr uint32_t WAIT_HINT_NS = 1000;
#ifndef POLL_SLEEP_NS
#define POLL_SLEEP_NS 100
#endif
constexpr int STATUS_TIMEOUT = 12;
constexpr uint32_t TMEM_COLS = 256;  // S of even pages: columns 0..63, of odd pages: 64..127; the output O: 128..128+DP-1
constexpr uint32_t S1_COL = 64, O_COL = 128;
constexpr float RESCALE_STEP = 8.f;  // the output is corrected only when a row's maximum has grown by more than this (base-2 units)
constexpr int LOADERS = 128;         // threads of warps 4-7, which copy the pages
constexpr int COPIER = 160;          // with TMA: the thread that issues the copies of the pages (first of warp 5)
constexpr int ISSUER = 128;          // the thread that issues the tensor-core products (first of warp 4)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_shared_16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// shared memory written by threads or cp.async becomes visible to the tensor core's reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
        __nanosleep(POLL_SLEEP_NS);      // a polling warp takes issue slots from the other CTA's working warps
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
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
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

// DP: head size padded to a multiple of 64 (the tensor core reads 64-element, 128-byte rows);
// the pad columns of Q, K and V are zero.
// TMA: the pages come by TMA (head sizes that are multiples of 64: a page of one head is then whole
// 64 x 64 boxes), issued by the thread that issues the products; otherwise warps 4-7 copy them
// with cp.async, 16 bytes a thread, which at this kernel's rate of pages is bound by the number
// of requests L2 takes.
template <int DP, bool TMA>
__global__ void __launch_bounds__(THREADS, 2) prefill_attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ tiles,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, __nv_bfloat16 *__restrict__ out, int ldo, int H, int Hkv, int D,
    int hpc, float scale, int window, int *__restrict__ status) {
    constexpr int KB = DP / 64;                       // 64-element blocks along the head dimension
    constexpr uint32_t Q_BYTES = KB * ROWS * 128;     // [KB][128 rows][128 B]
    constexpr uint32_t K_BYTES = KB * PAGE * 128;     // [KB][64 keys][128 B]      (K-major: row = key)
    constexpr uint32_t V_BYTES = KB * PAGE * 128;     // [KB][64 keys][128 B]      (N-major: 64 dims per row)
    constexpr uint32_t P_BYTES = ROWS * 128;          // [128 rows][64 keys]
    constexpr int HALF = DP / 2;                      // output columns per thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *Qs = base, *Ks = Qs + Q_BYTES, *Vs = Ks + 2 * K_BYTES, *Ps = Vs + V_BYTES;
    // [2][128] the page's correction of the running output, by the page's parity: a softmax warp
    // may be a page ahead of the warp that still adds up the page before
    float *corr_s = reinterpret_cast<float *>(Ps + P_BYTES);
    float *l_s = corr_s + 2 * ROWS;                             // [128] final sums
    __shared__ uint64_t s_bar, o_bar, k_full[2], v_full;
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
    const int n_iter = pg_hi - pg_lo + 1;
    const float scale_log2 = scale * 1.4426950408889634f;
    const int chunks_d = D / 8;                                   // 16-byte chunks of a real row

    if (tid == 0) {
        mbar_init(&s_bar, 1);
        mbar_init(&o_bar, 1);
        mbar_init(&k_full[0], 1);
        mbar_init(&k_full[1], 1);
        mbar_init(&v_full, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(&tmem_base_s, TMEM_COLS);
    // zero everything once: pad columns, rows of absent tokens and of heads this CTA does not have
    for (uint32_t i = tid * 16; i < Q_BYTES + 2 * K_BYTES + V_BYTES + P_BYTES; i += THREADS * 16)
        *reinterpret_cast<uint4 *>(base + i) = make_uint4(0, 0, 0, 0);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // ---- page copies ------------------------------------------------------------------------------
    // A page of one head is PAGE rows of chunks_d 16-byte chunks; loader thread l copies chunks l,
    // l + LOADERS, ...  Row and chunk of its first one are worked out once, the later ones
    // follow by addition (no division in the loop over pages).
    const int ltid = tid - LOADERS;                               // index among the loader threads (warps 4-7)
    const int row_first = ltid / chunks_d, ch_first = ltid - row_first * chunks_d;
    const int row_step = LOADERS / chunks_d, ch_step = LOADERS - row_step * chunks_d;
    // When the chunks of a row divide the loader threads, a thread keeps its chunk and moves down
    // row_step rows (a multiple of 8) each time: both addresses advance by constants.
    const bool linear = ch_step == 0;
    const uint32_t dst_first = (uint32_t)(ch_first >> 3) * (PAGE * 128) + swz(row_first, ch_first & 7);
    const int src_first = row_first * D + ch_first * 8;
    auto copy_page = [&](uint32_t dst, const __nv_bfloat16 *src, int valid_rows) {
        if (linear) {
            uint32_t d = dst + dst_first;
            const __nv_bfloat16 *sp = src + src_first;
            const uint32_t d_step = (uint32_t)row_step * 128;
            const int s_step = row_step * D;
#pragma unroll 4
            for (int row = row_first; row < PAGE; row += row_step) {
                cp_async_16(d, sp, row < valid_rows);
                d += d_step;
                sp += s_step;
            }
            return;
        }
        int row = row_first, ch = ch_first;
        while (row < PAGE) {
            cp_async_16(dst + (ch >> 3) * (PAGE * 128) + swz(row, ch & 7), src + row * D + ch * 8, row < valid_rows);
            row += row_step;
            ch += ch_step;
            if (ch >= chunks_d) {
                ch -= chunks_d;
                ++row;
            }
        }
    };
    auto load_k = [&](int it) {
        const int pg = pg_lo + it, stage = it & 1;
        const int page = table[pg];
        const bool have = page >= 0 && page < n_pages;
        if (ltid == 0 && !have) atomicExch(status, 3);
        const int valid_rows = have ? min(pos_last - pg * PAGE + 1, PAGE) : 0;   // rows past the last key become zero
        const size_t off = ((size_t)(have ? page : 0) * Hkv + kvh) * PAGE * D;
        const uint32_t dst = smem_u32(Ks + stage * K_BYTES);
        copy_page(dst, k_pages + off, valid_rows);
    };
    auto load_v = [&](int it) {
        const int pg = pg_lo + it;
        const int page = table[pg];
        const bool have = page >= 0 && page < n_pages;
        const int valid_rows = have ? min(pos_last - pg * PAGE + 1, PAGE) : 0;
        const size_t off = ((size_t)(have ? page : 0) * Hkv + kvh) * PAGE * D;
        const uint32_t dst = smem_u32(Vs);
        copy_page(dst, v_pages + off, valid_rows);
    };
    // The same by TMA (one thread): the page's 64 x 64 boxes; what it reads of rows past the last
    // key is dealt with where it matters (see the values below).
    auto tma_k = [&](int it) {
        const int page = table[pg_lo + it];
        const bool have = page >= 0 && page < n_pages;
        if (!have) atomicExch(status, 3);
        uint64_t *bar = &k_full[it & 1];
        mbar_expect_tx(bar, K_BYTES);
        for (int b = 0; b < KB; ++b) tma_load_box(smem_u32(Ks + (it & 1) * K_BYTES) + b * (PAGE * 128), &map_k, b * 64, (have ? page : 0) * Hkv + kvh, bar);
    };
    auto tma_v = [&](int it) {
        const int page = table[pg_lo + it];
        const bool have = page >= 0 && page < n_pages;
        mbar_expect_tx(&v_full, V_BYTES);
        for (int b = 0; b < KB; ++b) tma_load_box(smem_u32(Vs) + b * (PAGE * 128), &map_v, b * 64, (have ? page : 0) * Hkv + kvh, &v_full);
    };
    // The positions, tiles and block tables come from the host; everything else this kernel reads
    // (queries, this step's keys and values) is written by the kernels ahead of it.
    pdl_wait();
    const bool loader = !TMA && warp >= 4;    // without TMA warps 4-7 copy the pages; warps 0-3 do the softmax
    if (loader) {
        load_k(0);
        load_v(0);
        if (n_iter > 1) load_k(1);
        cp_async_commit();
    }
    if (TMA && tid == COPIER) {
        tma_k(0);
        tma_v(0);
        if (n_iter > 1) tma_k(1);
    }
    // queries: row r = token (r / hpc), head g0 + (r % hpc); through L2, they were just written
    for (int c = tid; c < ROWS * chunks_d; c += THREADS) {
        const int r = c / chunks_d, ch = c - r * chunks_d;
        const int tok = r / hpc, g = r - tok * hpc;
        if (tok < n_tok && g < g_count) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(q + (size_t)(row0 + tok) * ldq + (size_t)(kvh * group + g0 + g) * D + ch * 8));
            *reinterpret_cast<uint4 *>(Qs + (ch >> 3) * (ROWS * 128) + swz(r, ch & 7)) = v;
        }
    }

    // ---- per-thread state ---------------------------------------------------------------------------
    const int quarter = warp & 3;                                 // TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;                          // this thread's row
    const int my_tok = row / hpc, my_g = row - my_tok * hpc;
    const bool row_valid = my_tok < n_tok && my_g < g_count;
    const int qpos = row_valid ? pos_first + my_tok : -1;
    // m_ref: the maximum (base-2 units) that this row's sum l_run and its output in tensor memory
    // are relative to.  It follows the row's running maximum only when that has grown by more
    // than RESCALE_STEP since: until then the exponentials are taken against the older maximum
    // (they stay below 2^RESCALE_STEP) and the output needs no correction.
    float m_ref = -INFINITY, l_run = 0.f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    constexpr uint32_t idesc_qk = make_idesc(ROWS, PAGE, 0);
    constexpr uint32_t idesc_pv = make_idesc(ROWS, DP, 1);
    bool alive = true;

    // S = Q K^T of page `it` into the S buffer of its parity (one thread issues).  The descriptors
    // differ from their first one only in the address field (units of 16 bytes), so they are made
    // once and advanced by additions.
    const uint64_t desc_q0 = make_desc(smem_u32(Qs), 16, 1024), desc_k0 = make_desc(smem_u32(Ks), 16, 1024);
    const uint64_t desc_p0 = make_desc(smem_u32(Ps), 16, 1024), desc_v0 = make_desc(smem_u32(Vs), PAGE * 128, 1024);
    auto issue_qk = [&](int it) {
        const uint64_t dk = desc_k0 + (uint64_t)(((it & 1) * K_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < DP / 16; ++ks) {
            const uint64_t da = desc_q0 + (uint64_t)(((ks >> 2) * (ROWS * 128) + (ks & 3) * 32) >> 4);
            const uint64_t db = dk + (uint64_t)(((ks >> 2) * (PAGE * 128) + (ks & 3) * 32) >> 4);
            tcgen05_mma_bf16(tmem_base + ((it & 1) ? S1_COL : 0u), da, db, idesc_qk, ks > 0 ? 1u : 0u);
        }
        tcgen05_commit(&s_bar);
    };
    // Q and K(0) have landed: the first scores; later ones are issued a page ahead, behind the
    // P V product of the page before.
    cp_async_wait<0>();
    fence_async_smem();
    __syncthreads();
    if (tid == ISSUER) {
        if (TMA && alive && !mbar_wait(&k_full[0], 0, abort_flag, status)) alive = false;
        tcgen05_fence_after();
        issue_qk(0);
    }

    for (int it = 0; it < n_iter; ++it) {
        const int stage = it & 1, pg = pg_lo + it, key0 = pg * PAGE;
        const uint32_t s_col = stage ? S1_COL : 0u;
        int need = 0;

        // ---- softmax: warps 0-3, one thread per row, the page's scores in registers ---------------------
        if (warp < 4) {
            // (the scores of page it were issued behind P V of page it-1: once they are here, that
            //  product is done too and P may be written again)
            if (alive && !mbar_wait(&s_bar, it & 1, abort_flag, status)) alive = false;
            tcgen05_fence_after();
            const int page_id = table[pg];
            const bool have = page_id >= 0 && page_id < n_pages;
            // Columns c (keys key0 + c) this row may see: c_lo <= c <= c_hi.  A page that lies wholly
            // inside every row's range takes the path without per-element tests.
            // (rows without a token or a head hold zero queries: their scores are 0, their sums finite, and they are never written)
            const bool edge = !have || key0 + PAGE - 1 > pos_first || (window > 0 && key0 < pos_last - window + 1);
            const int c_hi = have ? qpos - key0 : -1;                                  // qpos = -1 for a row without a token
            const int c_lo = (window > 0) ? qpos - window + 1 - key0 : -(1 << 30);
            uint32_t r[PAGE];
#pragma unroll
            for (int c0 = 0; c0 < PAGE; c0 += 16) tcgen05_ld_16(lane_addr + s_col + (uint32_t)c0, *reinterpret_cast<uint32_t(*)[16]>(&r[c0]));
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
                for (int c = 0; c < PAGE; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(r[c]));
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
                need = 1;
            }
            corr_s[row] = corr;
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;    // keeps (-inf) - (-inf) out of the exponent
            // With TMA the next page's scores are issued ahead of P V, so their arrival says nothing
            // about that product: it must be done before P is written again (it mostly is by now).
            if (TMA && it > 0 && alive && !mbar_wait(&o_bar, (it - 1) & 1, abort_flag, status)) alive = false;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t p_row = smem_u32(Ps) + (uint32_t)((row >> 3) * 1024 + (row & 7) * 128);   // this row of P
            const uint32_t p_xor = (uint32_t)(row & 7);
            if (edge) {
#pragma unroll
                for (int c0 = 0; c0 < PAGE; c0 += 8) {
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        float p0 = ex2(fmaf(__uint_as_float(r[c0 + j]), scale_log2, neg_m));
                        float p1 = ex2(fmaf(__uint_as_float(r[c0 + j + 1]), scale_log2, neg_m));
                        if (c0 + j > c_hi || c0 + j < c_lo) p0 = 0.f;
                        if (c0 + j + 1 > c_hi || c0 + j + 1 < c_lo) p1 = 0.f;
                        sum4[(j >> 1) & 3] += p0 + p1;
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                        packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                    }
                    st_shared_16(p_row + ((((uint32_t)(c0 >> 3)) ^ p_xor) << 4), packed[0], packed[1], packed[2], packed[3]);
                }
            } else {
                // every row sees the whole page: no tests
#pragma unroll
                for (int c0 = 0; c0 < PAGE; c0 += 8) {
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(r[c0 + j]), scale_log2, neg_m));
                        const float p1 = ex2(fmaf(__uint_as_float(r[c0 + j + 1]), scale_log2, neg_m));
                        sum4[(j >> 1) & 3] += p0 + p1;
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                        packed[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                    }
                    st_shared_16(p_row + ((((uint32_t)(c0 >> 3)) ^ p_xor) << 4), packed[0], packed[1], packed[2], packed[3]);
                }
            }
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        }
        // V(it) and K(it+1) have landed (the loaders wait for their copies); P is written.  The
        // barrier also tells everyone whether any row's output has to be corrected first.
        cp_async_wait<0>();
        fence_async_smem();
        tcgen05_fence_before();
        const int any_need = __syncthreads_or(need);
        if (warp >= 4) {
            if (any_need) {
                // ---- correct the running output in tensor memory (rare): row by row, warps 4-7 ------------
                // (a correction implies an earlier page: its product into O must be done)
                if (alive && !mbar_wait(&o_bar, (it - 1) & 1, abort_flag, status)) alive = false;
                tcgen05_fence_after();
                const float corr = corr_s[row];
                // (tensor-memory loads and stores are for whole warps: a warp goes in if any of its rows needs it)
                if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                    for (int c0 = 0; c0 < DP; c0 += 16) {
                        uint32_t r[16];
                        tcgen05_ld_16(lane_addr + O_COL + (uint32_t)c0, r);
                        tcgen05_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
                        tcgen05_st_16(lane_addr + O_COL + (uint32_t)c0, r);
                    }
                    tcgen05_wait_st();
                }
                tcgen05_fence_before();
                asm volatile("bar.sync 1, 128;" ::: "memory");      // warps 4-7: all rows corrected before the product
            }
            if (TMA) {
                // ---- the scores of the next page, then O += P V, then the next copies: warp 4 ---------------
                // (the scores first: the next softmax waits for them and they need nothing of this one)
                if (warp == 4) {
                    if (lane == 0) {
                        tcgen05_fence_after();
                        if (it + 1 < n_iter) {
                            if (alive && !mbar_wait(&k_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_flag, status)) alive = false;
                            issue_qk(it + 1);
                        }
                        if (alive && !mbar_wait(&v_full, it & 1, abort_flag, status)) alive = false;
                    }
                    __syncwarp();
                    // The values of rows past the tile's last key (the rest of its last page, or a
                    // page the table does not hold) may be anything, NaN included, and 0 x NaN is NaN:
                    // they become zeros.  (Keys there give scores that the softmax masks.)
                    const int page = table[pg];
                    const int valid_rows = (page >= 0 && page < n_pages) ? min(pos_last - pg * PAGE + 1, PAGE) : 0;
                    if (valid_rows < PAGE) {
                        for (int i = lane; i < (PAGE - valid_rows) * chunks_d; i += 32) {
                            const int zr = valid_rows + i / chunks_d, ch = i % chunks_d;
                            st_shared_16(smem_u32(Vs) + (ch >> 3) * (PAGE * 128) + swz(zr, ch & 7), 0u, 0u, 0u, 0u);
                        }
                        fence_async_smem();
                        __syncwarp();
                    }
                    if (lane == 0) {
#pragma unroll
                        for (int k2 = 0; k2 < PAGE / 16; ++k2)
                            tcgen05_mma_bf16(tmem_base + O_COL, desc_p0 + (uint64_t)((k2 * 32) >> 4), desc_v0 + (uint64_t)((k2 * 2048) >> 4), idesc_pv,
                                             (it > 0 || k2 > 0) ? 1u : 0u);
                        tcgen05_commit(&o_bar);
                    }
                    __syncwarp();
                } else if (tid == COPIER) {
                    // ---- the next copies, by a thread of their own (issuing a product or a copy
                    // takes the issuing thread tens of cycles each: one thread for both was the
                    // slowest part of a page) ----
                    // the keys' stage of this page is free (its scores were seen before the barrier)
                    if (it + 2 < n_iter) tma_k(it + 2);
                    // the values' stage is free once the product has read it
                    if (alive && !mbar_wait(&o_bar, it & 1, abort_flag, status)) alive = false;
                    if (it + 1 < n_iter) tma_v(it + 1);
                }
                continue;
            }
            // ---- O += P V, and the scores of the next page behind it ---------------------------------------
            if (tid == ISSUER) {
                tcgen05_fence_after();
#pragma unroll
                for (int k2 = 0; k2 < PAGE / 16; ++k2) {
                    // 16 keys further: 32 bytes along a row of P; two groups of 8 rows of V (blocks of 64
                    // dims are PAGE * 128 bytes apart: the leading offset of the V descriptor)
                    tcgen05_mma_bf16(tmem_base + O_COL, desc_p0 + (uint64_t)((k2 * 32) >> 4), desc_v0 + (uint64_t)((k2 * 2048) >> 4), idesc_pv,
                                     (it > 0 || k2 > 0) ? 1u : 0u);
                }
                tcgen05_commit(&o_bar);
                if (it + 1 < n_iter) issue_qk(it + 1);
            }
            // The softmax warps saw the scores of this page before the barrier above, so its keys' stage
            // is free: the keys of the page after the next.
            if (it + 2 < n_iter) load_k(it + 2);
            // the values' stage is free once the product has read it: the next page of values
            if (alive && !mbar_wait(&o_bar, it & 1, abort_flag, status)) alive = false;
            if (it + 1 < n_iter) load_v(it + 1);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    // ---- normalise and write: every thread half the columns of its row -------------------------------------
    if (warp < 4) {
        l_s[row] = l_run;
        // the loaders waited for the last product; the softmax warps have not yet
        if (alive && n_iter > 0 && !mbar_wait(&o_bar, (n_iter - 1) & 1, abort_flag, status)) alive = false;
    }
    tcgen05_fence_after();
    __syncthreads();
    {
        // (every lane takes part in the loads from tensor memory, which are for whole warps; rows
        //  without a token only skip the stores)
        const float l = l_s[row];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int col0 = warp < 4 ? 0 : HALF;
        const bool store = row_valid && alive;
        __nv_bfloat16 *dst = out + (size_t)(row0 + (store ? my_tok : 0)) * ldo + (size_t)(kvh * group + g0 + (store ? my_g : 0)) * D;
#pragma unroll
        for (int c0 = 0; c0 < HALF; c0 += 16) {
            uint32_t r[16];
            tcgen05_ld_16(lane_addr + O_COL + (uint32_t)(col0 + c0), r);
            tcgen05_wait_ld();
#pragma unroll
            for (int c8 = 0; c8 < 16; c8 += 8) {
                const int d = col0 + c0 + c8;
                if (store && d + 8 <= D) {
                    uint32_t h[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(r[c8 + 2 * j]) * inv, __uint_as_float(r[c8 + 2 * j + 1]) * inv);
                        h[j] = *reinterpret_cast<uint32_t *>(&pr);
                    }
                    *reinterpret_cast<uint4 *>(dst + d) = make_uint4(h[0], h[1], h[2], h[3]);
                }
            }
        }
    }
    tcgen05_fence_before();
    pdl_trigger();      // at the end, as in the two-tile kernel: a CTA that fills its SM keeps the next kernel back until it is done
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------------
// LGML_ATTN_TMA=0: the pages are always copied with cp.async.
bool tma_pages_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("LGML_ATTN_TMA");
        on = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

template <int DP, bool TMA>
int launch(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *tiles, const int *block_table, int max_blocks,
           const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo, int H, int Hkv, int D,
           int hpc, float scale, int window, int *status, cudaStream_t stream) {
    constexpr int KB = DP / 64;
    const size_t smem = (size_t)KB * ROWS * 128 + 3 * (size_t)KB * PAGE * 128 + ROWS * 128 + 3 * ROWS * sizeof(float) + 1024;
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<DP, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) LGML_FAIL("prefill_attention_tc: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    CUtensorMap mk, mv;
    memset(&mk, 0, sizeof(mk));
    memset(&mv, 0, sizeof(mv));
    if (TMA) {
        int rc;
        if ((rc = lgml_make_page_map(&mk, k_pages, n_pages, Hkv, D, "prefill_attention_tc"))) return rc;
        if ((rc = lgml_make_page_map(&mv, v_pages, n_pages, Hkv, D, "prefill_attention_tc"))) return rc;
    }
    lgml_launch(prefill_attention_tc_kernel<DP, TMA>, grid, THREADS, smem, stream, mk, mv, q, ldq, positions, tiles, block_table, max_blocks,
                k_pages, v_pages, n_pages, out, ldo, H, Hkv, D, hpc, scale, window, status);
    return lgml_launch_status("prefill_attention_tc");
}
}  // namespace

// Heads per CTA for a group of `group` query heads per KV head (at most 8) and the tokens of a
// tile: 128 rows / heads per CTA.
LGML_API void lgml_prefill_attention_tc_shape(int group, int *heads_per_cta, int *tile_tokens) {
    const int hpc = group < 8 ? group : 8;
    *heads_per_cta = hpc;
    *tile_tokens = ROWS / hpc;
}

LGML_API int lgml_prefill_attention_tc(const void *q, int ldq, const int *positions, const int *tiles, int n_tiles, const int *block_table,
                                       int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, void *out,
                                       int ldo, int H, int Hkv, int D, float scale, int window, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tiles >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "prefill_attention_tc: bad sizes");
    LGML_REQUIRE(page_size == PAGE, "prefill_attention_tc: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0, "prefill_attention_tc: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D >= 16 && D <= 128 && D % 16 == 0, "prefill_attention_tc: head_dim %d must be a multiple of 16 up to 128", D);
    LGML_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 && D % 8 == 0,
                 "prefill_attention_tc: q and out must be 16-byte aligned with row strides that are multiples of 8");
    LGML_REQUIRE(((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0, "prefill_attention_tc: the cache must be 16-byte aligned");
    if (n_tiles == 0) return 0;
    const int group = H / Hkv;
    int hpc, tt;
    lgml_prefill_attention_tc_shape(group, &hpc, &tt);
    const int chunks = (group + hpc - 1) / hpc;
    LGML_REQUIRE((long long)Hkv * chunks <= 65535, "prefill_attention_tc: too many heads");
    LGML_REQUIRE(n_tiles <= 65535, "prefill_attention_tc: %d tiles in one launch (at most 65535)", n_tiles);
    dim3 grid(Hkv * chunks, n_tiles);
    const __nv_bfloat16 *qq = (const __nv_bfloat16 *)q, *kk = (const __nv_bfloat16 *)k_pages, *vv = (const __nv_bfloat16 *)v_pages;
    __nv_bfloat16 *oo = (__nv_bfloat16 *)out;
#define LGML_ARGS grid, qq, ldq, positions, tiles, block_table, max_blocks, kk, vv, n_pages, oo, ldo, H, Hkv, D, hpc, scale, window, status, stream
    const bool tma = tma_pages_enabled() && D % 64 == 0;     // a page of one head is then whole 64 x 64 boxes
    if (D <= 64) return tma ? launch<64, true>(LGML_ARGS) : launch<64, false>(LGML_ARGS);
    return tma ? launch<128, true>(LGML_ARGS) : launch<128, false>(LGML_ARGS);
#undef LGML_ARGS
}
