// Paged attention for prompts and portions of prompts (many query tokens per request),
// bfloat16 with float32 softmax, on tensor cores.
//
// A CTA takes one tile of a request's new tokens (up to 16 * n_tb consecutive tokens) and the
// query heads that share one KV head (up to `hpc` of them); warp w works on 16 tokens of one
// head: its 16 x D block of Q lives in registers as matrix fragments for the whole kernel.
// The CTA walks the request's pages from the first one a query can see to the page of its
// last token: a page of K and of V (64 x D each) is copied into shared memory with cp.async
// (two stages, so the next page is in flight while this one is used) and shared by all warps,
// so grouped heads read each page from HBM once.  Per page and warp: S = Q K^T (16 x 64) by
// mma.sync m16n8k16, scale, causal/window mask from the positions, online softmax in float32
// (running maximum and sum per row), P rounded to bfloat16 as the A operand of O += P V.
// Keys are taken from the cache, so this step's own keys are seen at cache precision, as in
// mischief/lgml, which writes the cache before attention reads it
// (lua/lgml/transformer.lua:1838-1839, :2405-2407; formula :1805-1816, scale :1845).
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_prefill)

namespace {
constexpr int PAGE = 64;
constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void *dst, const void *src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// tiles: [n_tiles][4] = (request row in the batch, first token row, tokens in the tile, unused)
template <int D>
__global__ void __launch_bounds__(THREADS, 1) prefill_attention_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ tiles,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, __nv_bfloat16 *__restrict__ out, int ldo, int H, int Hkv,
    int hpc, int n_tb, float scale, int window, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    constexpr int LD = D + 8;                    // padded row of the shared tiles (elements): ldmatrix without bank conflicts
    constexpr int KS = D / 16;                   // k steps of Q K^T
    constexpr int DT = D / 8;                    // n tiles of the output
    constexpr int CHUNKS = PAGE * (D / 8);       // 16-byte chunks of one page of K (or V)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16 *kv_s = reinterpret_cast<__nv_bfloat16 *>(smem_raw);   // [2 stages][K | V][PAGE][LD]
    __shared__ int page_ok[2];

    const int tile = blockIdx.y;                  // heads run fastest: the CTAs of one tile start together, tiles in the order given
    const int seq = tiles[tile * 4 + 0], row0 = tiles[tile * 4 + 1], n_tok = tiles[tile * 4 + 2];
    const int group = H / Hkv;
    const int chunks_per_kv = (group + hpc - 1) / hpc;
    const int kvh = blockIdx.x / chunks_per_kv, hchunk = blockIdx.x - kvh * chunks_per_kv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head_local = warp % hpc, tb = warp / hpc;
    const int g = hchunk * hpc + head_local;                      // head within the group
    const bool warp_active = tb < n_tb && g < group && tb * 16 < n_tok;
    const int h = kvh * group + g;
    const int *table = block_table + (size_t)seq * max_blocks;

    const int pos_first = positions[row0], pos_last = pos_first + n_tok - 1;
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int pg_lo = lo_first / PAGE, pg_hi = pos_last / PAGE;
    const float scale_log2 = scale * 1.4426950408889634f;

    // ---- this warp's queries as A fragments -----------------------------------------------------
    const int r_in = lane >> 2, c_in = (lane & 3) * 2;
    const int wrow0 = tb * 16;                                    // first token of the warp within the tile
    const int rows_valid = warp_active ? min(16, n_tok - wrow0) : 0;
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r_in + (i & 1) * 8, d = ks * 16 + c_in + (i >> 1) * 8;
            uint32_t v = 0;
            if (r < rows_valid) v = act_load(reinterpret_cast<const unsigned int *>(q + (size_t)(row0 + wrow0 + r) * ldq + (size_t)h * D + d));
            qf[ks][i] = v;
        }
    }
    float oacc[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int qpos[2] = {r_in < rows_valid ? pos_first + wrow0 + r_in : -1, r_in + 8 < rows_valid ? pos_first + wrow0 + r_in + 8 : -1};

    // ---- page loads --------------------------------------------------------------------------------
    auto load_page = [&](int pg, int stage) {
        const int page = table[pg];
        const bool have = page >= 0 && page < n_pages;
        if (tid == 0) {
            page_ok[stage] = have ? 1 : 0;
            if (!have) atomicExch(status, 3);
        }
        const int valid_rows = have ? min(pos_last - pg * PAGE + 1, PAGE) : 0;   // rows past the last key stay zero
        const size_t off = ((size_t)(have ? page : 0) * Hkv + kvh) * PAGE * D;
        __nv_bfloat16 *ks_ = kv_s + (size_t)stage * 2 * PAGE * LD, *vs_ = ks_ + PAGE * LD;
        for (int c = tid; c < CHUNKS; c += THREADS) {
            const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
            const bool ok = row < valid_rows;
            cp_async_16(ks_ + row * LD + col, k_pages + off + (size_t)row * D + col, ok);
            cp_async_16(vs_ + row * LD + col, v_pages + off + (size_t)row * D + col, ok);
        }
        cp_async_commit();
    };

    load_page(pg_lo, 0);
    for (int pg = pg_lo; pg <= pg_hi; ++pg) {
        const int stage = (pg - pg_lo) & 1;
        if (pg + 1 <= pg_hi) {
            load_page(pg + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16 *ks_ = kv_s + (size_t)stage * 2 * PAGE * LD, *vs_ = ks_ + PAGE * LD;
        const int key0 = pg * PAGE;
        // a warp whose queries all lie before this page has nothing to see in it
        const bool needed = warp_active && page_ok[stage] && key0 <= pos_first + wrow0 + rows_valid - 1;
        if (needed) {
            // ---- S = Q K^T -------------------------------------------------------------------------
            float sacc[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
            const int mat = lane >> 3, mrow = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int nt = 0; nt < 8; nt += 2) {
                    uint32_t b[4];
                    ldmatrix_x4(b, ks_ + (size_t)((nt + (mat >> 1)) * 8 + mrow) * LD + ks * 16 + (mat & 1) * 8);
                    mma_bf16(sacc[nt], qf[ks], b[0], b[1]);
                    mma_bf16(sacc[nt + 1], qf[ks], b[2], b[3]);
                }
            }
            // ---- scale, mask, online softmax -----------------------------------------------------------
            const bool edge = key0 + PAGE - 1 > pos_first + wrow0 || (window > 0 && key0 < pos_first + wrow0 + 15 - window + 1);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1;
                    float s = sacc[nt][i] * scale_log2;   // base-2 domain: exp(x) = exp2(x log2 e)
                    if (edge) {
                        const int kpos = key0 + nt * 8 + c_in + (i & 1);
                        if (kpos > qpos[rr] || (window > 0 && kpos < qpos[rr] - window + 1)) s = -INFINITY;
                    } else if (qpos[rr] < 0) {
                        s = -INFINITY;
                    }
                    sacc[nt][i] = s;
                    mx[rr] = fmaxf(mx[rr], s);
                }
            }
            float corr[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
                const float m_new = fmaxf(m_run[rr], mx[rr]);
                corr[rr] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[rr] - m_new);
                m_run[rr] = m_new;
                l_run[rr] *= corr[rr];
            }
            uint32_t pf[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float p[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1;
                    p[i] = (m_run[rr] == -INFINITY) ? 0.f : exp2f(sacc[nt][i] - m_run[rr]);
                    l_run[rr] += p[i];
                }
                // the C layout of S is the A layout of P: two n tiles of 8 keys make one k step of 16
                pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
            }
#pragma unroll
            for (int dt = 0; dt < DT; ++dt) {
                oacc[dt][0] *= corr[0];
                oacc[dt][1] *= corr[0];
                oacc[dt][2] *= corr[1];
                oacc[dt][3] *= corr[1];
            }
            // ---- O += P V ------------------------------------------------------------------------------
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2) {
#pragma unroll
                for (int dt = 0; dt < DT; dt += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vs_ + (size_t)(k2 * 16 + (mat & 1) * 8 + mrow) * LD + dt * 8 + (mat >> 1) * 8);
                    mma_bf16(oacc[dt], pf[k2], b[0], b[1]);
                    mma_bf16(oacc[dt + 1], pf[k2], b[2], b[3]);
                }
            }
        }
        __syncthreads();   // the stage may be overwritten by the load two pages ahead
    }

    // ---- normalise and write ---------------------------------------------------------------------------
    if (warp_active) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
            l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int r = r_in + rr * 8;
            if (r >= rows_valid) continue;
            const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
            __nv_bfloat16 *dst = out + (size_t)(row0 + wrow0 + r) * ldo + (size_t)h * D;
#pragma unroll
            for (int dt = 0; dt < DT; ++dt)
                *reinterpret_cast<uint32_t *>(dst + dt * 8 + c_in) = pack_bf16(oacc[dt][rr * 2] * inv, oacc[dt][rr * 2 + 1] * inv);
        }
    }
}

template <int D>
int launch(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *tiles, const int *block_table, int max_blocks,
           const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo, int H, int Hkv, int hpc,
           int n_tb, float scale, int window, int *status, cudaStream_t stream) {
    const size_t smem = (size_t)2 * 2 * PAGE * (D + 8) * sizeof(__nv_bfloat16);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("prefill_attention: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(prefill_attention_kernel<D>, grid, THREADS, smem, stream, q, ldq, positions, tiles, block_table, max_blocks, k_pages,
                v_pages, n_pages, out, ldo, H, Hkv, hpc, n_tb, scale, window, status);
    return lgml_launch_status("prefill_attention");
}
}  // namespace

// How a CTA's 8 warps are split for a group of `group` query heads per KV head: heads per CTA
// (at most 8) and blocks of 16 tokens; a tile holds 16 * n_tb tokens.
LGML_API void lgml_prefill_attention_shape(int group, int *heads_per_cta, int *token_blocks) {
    int hpc = group < WARPS ? group : WARPS;
    *heads_per_cta = hpc;
    *token_blocks = WARPS / hpc;
}

LGML_API int lgml_prefill_attention(const void *q, int ldq, const int *positions, const int *tiles, int n_tiles, const int *block_table,
                                    int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, void *out,
                                    int ldo, int H, int Hkv, int D, float scale, int window, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tiles >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "prefill_attention: bad sizes");
    LGML_REQUIRE(page_size == PAGE, "prefill_attention: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0, "prefill_attention: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D >= 16 && D <= 128 && D % 16 == 0, "prefill_attention: head_dim %d must be a multiple of 16 up to 128", D);
    LGML_REQUIRE(ldq % 2 == 0 && ldo % 2 == 0 && ((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 3) == 0, "prefill_attention: q and out must be 4-byte aligned with even row strides");
    LGML_REQUIRE(((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0, "prefill_attention: the cache must be 16-byte aligned");
    if (n_tiles == 0) return 0;
    const int group = H / Hkv;
    int hpc, n_tb;
    lgml_prefill_attention_shape(group, &hpc, &n_tb);
    const int chunks = (group + hpc - 1) / hpc;
    LGML_REQUIRE((long long)Hkv * chunks <= 65535, "prefill_attention: too many heads");
    LGML_REQUIRE(n_tiles <= 65535, "prefill_attention: %d tiles in one launch (at most 65535)", n_tiles);
    dim3 grid(Hkv * chunks, n_tiles);
    const __nv_bfloat16 *qq = (const __nv_bfloat16 *)q, *kk = (const __nv_bfloat16 *)k_pages, *vv = (const __nv_bfloat16 *)v_pages;
    __nv_bfloat16 *oo = (__nv_bfloat16 *)out;
#define LGML_CASE(DD)                                                                                                                 \
    case DD:                                                                                                                          \
        return launch<DD>(grid, qq, ldq, positions, tiles, block_table, max_blocks, kk, vv, n_pages, oo, ldo, H, Hkv, hpc, n_tb, scale, \
                          window, status, stream);
    switch (D) {
        LGML_CASE(16) LGML_CASE(32) LGML_CASE(48) LGML_CASE(64) LGML_CASE(80) LGML_CASE(96) LGML_CASE(112) LGML_CASE(128)
    }
#undef LGML_CASE
    LGML_FAIL("prefill_attention: head_dim %d not handled", D);
}
