// Paged attention for decoding (and short portions), bfloat16 cache, float32 softmax, on
// tensor cores.
//
// Every query token is independent: token t of request s at position p attends to the
// cells of s at positions <= p (the last `window` of them if a window is set).  The work of
// one token is cut by KV head and, along the keys, into `n_splits` ranges of whole pages;
// one CTA handles (token, KV head [x chunk of up to 8 of its query heads], split).  The query
// heads that share a KV head (grouped-query attention) are processed together, so each key
// and value is read from HBM once for all of them.  A split leaves an unnormalised partial
// result (running maximum m, sum l, weighted values O) in scratch memory; a second kernel
// merges the splits in a fixed order.  With one split the result is written directly.
//
// With one query per head there is no tall Q tile, so the products are turned round: the keys
// are the M side of the tensor-core tile and the (up to 8) heads the N side:
//     S^T[64 keys, 8 heads] = K[64, D] . Q^T[D, 8]        (mma.sync m16n8k16, 4 x D/16 per page)
//     O^T[D, 8 heads]      += V^T[D, 64] . P^T[64, 8]      (D/16 x 4 per page)
// K is read row-major as the A operand (ldmatrix), V transposed (ldmatrix.trans), Q^T sits in
// registers for the whole kernel and P^T goes through shared memory as bfloat16.  Pages are
// copied into padded shared-memory rows with cp.async, three stages deep (two for head sizes
// over 128), so the copies of the next pages overlap the math of this one.  Softmax, the
// running sums and the output accumulators are float32 (lua/lgml/transformer.lua:1805-1816
// for the formula, :1845 for the scale).
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_decode)

namespace {
constexpr int PAGE = 64;
constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int MAX_D = 256;
constexpr int NH = 8;                  // heads per CTA = the N of the tensor-core tile

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

// KS = D / 16.  Each of the four warps is a pipeline of its own: of every page it copies,
// scores and weighs only its quarter of the keys (16), keeping a running maximum, sum and
// output of its own, so the loop over pages needs no barrier between warps; the four partial
// results are merged once at the end.
template <int KS, int STAGES>
__global__ void __launch_bounds__(THREADS) decode_attention_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, __nv_bfloat16 *__restrict__ out, int ldo,
    float *__restrict__ part_o, float2 *__restrict__ part_ml, int n_splits, int H, int Hkv, int heads_per_cta, int n_chunks,
    float scale, int window, int newest, int *__restrict__ status) {
    pdl_trigger();
    constexpr int D = KS * 16;
    constexpr int LD = D + 8;                       // padded row of the K and V stages (elements)
    constexpr int WK = PAGE / WARPS;                // keys of a page per warp: 16
    constexpr int PW = WK + 8;                      // padded row of a warp's P^T (bfloat16)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // per warp: [STAGES][K | V][WK][LD] bfloat16, then P^T [NH][PW] bfloat16
    constexpr size_t WARP_STAGE = (size_t)2 * WK * LD;                  // elements of one stage of one warp
    constexpr size_t WARP_BYTES = (STAGES * WARP_STAGE + NH * PW) * 2;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __nv_bfloat16 *kv_w = reinterpret_cast<__nv_bfloat16 *>(smem_raw + (size_t)warp * WARP_BYTES);
    __nv_bfloat16 *Pw = kv_w + STAGES * WARP_STAGE;

    const int t = blockIdx.x;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    const int split = blockIdx.z;
    const int group = H / Hkv;
    const int h0 = kvh * group + chunk * heads_per_cta;                 // first query head of this CTA
    const int g_count = min(heads_per_cta, group - chunk * heads_per_cta);
    const int mat = lane >> 3, mrow = lane & 7;

    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int *table = block_table + (size_t)seq * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_pages_seq = pos / PAGE + 1;
    const int first_page = lo / PAGE;
    const int span = n_pages_seq - first_page;
    const int pps = (span + n_splits - 1) / n_splits;
    const int pb = first_page + split * pps;
    const int pe = min(pb + pps, n_pages_seq);
    const int n_iter = max(pe - pb, 0);
    const float scale_log2 = scale * 1.4426950408889634f;   // scores in the base-2 domain: exp(x) = exp2(x log2 e)

    // Copy this warp's 16 rows of the page of iteration `it` into its stage it % STAGES; rows past
    // the last visible key, and a page the table does not hold, become zeros.
    auto load_rows = [&](int it) {
        const int pg = pb + it;
        const int page = table[pg];
        const bool have = page >= 0 && page < n_pages;
        if (!have && lane == 0) atomicExch(status, 3);
        const int valid_rows = have ? min(pos - pg * PAGE + 1, PAGE) : 0;
        const size_t off = ((size_t)(have ? page : 0) * Hkv + kvh) * PAGE * D + (size_t)warp * WK * D;
        __nv_bfloat16 *ks_ = kv_w + (size_t)(it % STAGES) * WARP_STAGE, *vs_ = ks_ + WK * LD;
#pragma unroll
        for (int c = lane; c < WK * (D / 8); c += 32) {
            const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
            const bool ok = warp * WK + row < valid_rows;
            cp_async_16(ks_ + row * LD + col, k_pages + off + (size_t)row * D + col, ok);
            cp_async_16(vs_ + row * LD + col, v_pages + off + (size_t)row * D + col, ok);
        }
    };
    // The positions and block tables come from the host, and pages that lie wholly before this
    // step's new tokens were written by earlier steps: their copies can start before the
    // kernels ahead of this one in the stream (which write this step's keys and the queries)
    // have finished.  `newest` is the most tokens any request brings in this step.
    const int old_pages = max(pos - newest + 1, 0) / PAGE;       // pages below this index hold old tokens only
    bool waited = false;
#pragma unroll
    for (int it = 0; it < STAGES - 1; ++it) {
        if (it < n_iter) {
            if (!waited && pb + it >= old_pages) {
                pdl_wait();
                waited = true;
            }
            load_rows(it);
        }
        cp_async_commit();
    }
    if (!waited) pdl_wait();

    // Q^T as B fragments: b0 holds (d = 16 ks + 2 (lane % 4) + {0, 1}, head = lane / 4), b1 the same 8 dims on
    uint32_t qb[KS][2];
    {
        const int head = lane >> 2;
        const __nv_bfloat16 *qrow = q + (size_t)t * ldq + (size_t)(h0 + head) * D + (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            // the queries were written by the kernel just ahead, while this one may already have been
            // running: read them through L2 (ld.global.cg), not through a cache that is only
            // coherent at kernel boundaries
            qb[ks][0] = head < g_count ? act_load(reinterpret_cast<const unsigned int *>(qrow + ks * 16)) : 0u;
            qb[ks][1] = head < g_count ? act_load(reinterpret_cast<const unsigned int *>(qrow + ks * 16 + 8)) : 0u;
        }
    }

    // this thread's two heads: columns (lane % 4) * 2 and + 1 of the S^T and O^T fragments
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[KS][4];
#pragma unroll
    for (int i = 0; i < KS; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

    for (int it = 0; it < n_iter; ++it) {
        if (it + STAGES - 1 < n_iter) load_rows(it + STAGES - 1);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const int pg = pb + it;
        const __nv_bfloat16 *ks_ = kv_w + (size_t)(it % STAGES) * WARP_STAGE, *vs_ = ks_ + WK * LD;
        const int key_base = pg * PAGE + warp * WK;               // position of this warp's first key

        // ---- S^T = K Q^T for the warp's 16 keys ---------------------------------------------------
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, ks_ + (size_t)((mat & 1) * 8 + mrow) * LD + ks * 16 + (mat >> 1) * 8);
            mma_bf16(c, a, qb[ks][0], qb[ks][1]);
        }
        // rows of the fragment are keys (lane / 4, + 8), columns heads ((lane % 4) * 2, + 1)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kpos = key_base + (lane >> 2) + (i >> 1) * 8;
            c[i] = (kpos >= lo && kpos <= pos) ? c[i] * scale_log2 : -INFINITY;
            mx[i & 1] = fmaxf(mx[i & 1], c[i]);
        }
        float corr[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 4));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 8));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 16));
            const float m_new = fmaxf(m_run[hh], mx[hh]);
            corr[hh] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[hh] - m_new);
            m_run[hh] = m_new;
        }
        // P^T through the warp's own shared memory: written as (head, key), read as B fragments
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int hh = i & 1;
            const float pf = (m_run[hh] == -INFINITY) ? 0.f : exp2f(c[i] - m_run[hh]);
            const __nv_bfloat16 ph = __float2bfloat16_rn(pf);
            // the sum runs over the probabilities as the product will see them (rounded to bfloat16)
            l_run[hh] = (i < 2 ? l_run[hh] * corr[hh] : l_run[hh]) + __bfloat162float(ph);
            Pw[((lane & 3) * 2 + hh) * PW + (lane >> 2) + (i >> 1) * 8] = ph;
        }
        __syncwarp();
        const uint32_t pb0 = *reinterpret_cast<const uint32_t *>(Pw + (lane >> 2) * PW + (lane & 3) * 2);
        const uint32_t pb1 = *reinterpret_cast<const uint32_t *>(Pw + (lane >> 2) * PW + (lane & 3) * 2 + 8);

        // ---- O^T += V^T P^T over the warp's 16 keys: one k step per 16-dim tile ---------------------
#pragma unroll
        for (int mt = 0; mt < KS; ++mt) {
            oacc[mt][0] *= corr[0];
            oacc[mt][1] *= corr[1];
            oacc[mt][2] *= corr[0];
            oacc[mt][3] *= corr[1];
            uint32_t a[4];
            ldmatrix_x4_trans(a, vs_ + (size_t)((mat >> 1) * 8 + mrow) * LD + mt * 16 + (mat & 1) * 8);
            mma_bf16(oacc[mt], a, pb0, pb1);
        }
    }
    cp_async_wait<0>();

    // ---- merge the four warps -----------------------------------------------------------------------
    // the sums: over the 8 lanes that share this thread's two heads
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
    }
    __syncthreads();                                             // every warp is done with its stages
    float *mo = reinterpret_cast<float *>(smem_raw);             // [WARPS][D][NH] outputs, then [WARPS][NH] m and l
    float *mm = mo + (size_t)WARPS * D * NH, *ml = mm + WARPS * NH;
#pragma unroll
    for (int mt = 0; mt < KS; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = mt * 16 + (lane >> 2) + (i >> 1) * 8, head = (lane & 3) * 2 + (i & 1);
            mo[((size_t)warp * D + d) * NH + head] = oacc[mt][i];
        }
    if (lane < 4) {
        mm[warp * NH + lane * 2] = m_run[0];
        mm[warp * NH + lane * 2 + 1] = m_run[1];
        ml[warp * NH + lane * 2] = l_run[0];
        ml[warp * NH + lane * 2 + 1] = l_run[1];
    }
    __syncthreads();
    for (int i = tid; i < D * NH; i += THREADS) {
        const int d = i / NH, head = i - d * NH;
        if (head >= g_count) continue;
        float m = -INFINITY;
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, mm[w * NH + head]);
        float o = 0.f, l = 0.f;
        for (int w = 0; w < WARPS; ++w) {
            const float f = (mm[w * NH + head] == -INFINITY) ? 0.f : exp2f(mm[w * NH + head] - m);
            o += mo[((size_t)w * D + d) * NH + head] * f;
            l += ml[w * NH + head] * f;
        }
        const int h = h0 + head;
        if (n_splits == 1) {
            out[(size_t)t * ldo + (size_t)h * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            part_o[(((size_t)t * H + h) * n_splits + split) * D + d] = o;
            if (d == 0) part_ml[((size_t)t * H + h) * n_splits + split] = make_float2(m * 0.6931471805599453f, l);   // the maximum back in natural units
        }
    }
}

// Merge the splits of one (token, head) in split order.  A thread adds up one dimension.  The
// loads of its first sixteen splits' partial outputs go out together with those of the splits'
// maxima and sums, before anything is computed (one after the other, every load would cost a round
// trip to L2: at batch 1 there are sixteen splits), and a split's factor exp(m - max) is computed
// once, by one thread, not by every thread for every split.
constexpr int MAX_SPLITS = 512;
constexpr int COMBINE_FIRST = 16;
__global__ void decode_combine_kernel(const float *__restrict__ part_o, const float2 *__restrict__ part_ml,
                                      __nv_bfloat16 *__restrict__ out, int ldo, int n_splits, int H, int D) {
    pdl_trigger();
    pdl_wait();
    __shared__ float m_s[MAX_SPLITS], w_s[MAX_SPLITS], f_s[MAX_SPLITS];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const float2 *ml = part_ml + ((size_t)t * H + h) * n_splits;
    const float *po = part_o + ((size_t)t * H + h) * n_splits * D;
    float first[COMBINE_FIRST];
#pragma unroll
    for (int u = 0; u < COMBINE_FIRST; ++u)
        if (u < n_splits && tid < D) first[u] = act_load(po + (size_t)u * D + tid);
    for (int i = tid; i < n_splits; i += blockDim.x) {
        const float2 v = act_load(ml + i);
        m_s[i] = v.x;
        w_s[i] = v.y;
    }
    __syncthreads();
    float mm = -INFINITY;
    for (int i = 0; i < n_splits; ++i) mm = fmaxf(mm, m_s[i]);
    for (int i = tid; i < n_splits; i += blockDim.x) f_s[i] = m_s[i] == -INFINITY ? 0.f : expf(m_s[i] - mm);
    __syncthreads();
    float l = 0.f;
    for (int i = 0; i < n_splits; ++i) l += m_s[i] == -INFINITY ? 0.f : w_s[i] * f_s[i];
    for (int d = tid; d < D; d += blockDim.x) {
        float o = 0.f;
        int i0 = 0;
        if (d == tid) {
#pragma unroll
            for (int u = 0; u < COMBINE_FIRST; ++u)
                if (u < n_splits && m_s[u] != -INFINITY) o += first[u] * f_s[u];
            i0 = COMBINE_FIRST;
        }
        for (; i0 < n_splits; i0 += 8) {
            float pv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + u < n_splits) pv[u] = act_load(po + (size_t)(i0 + u) * D + d);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + u < n_splits && m_s[i0 + u] != -INFINITY) o += pv[u] * f_s[i0 + u];
        }
        out[(size_t)t * ldo + (size_t)h * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

template <int KS, int STAGES>
int launch_ks(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
              int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo,
              float *part_o, float2 *part_ml, int n_splits, int H, int Hkv, int heads_per_cta, int n_chunks, float scale, int window,
              int newest, int *status, cudaStream_t stream) {
    constexpr int D = KS * 16;
    // per warp: its quarter of the K and V stages and its P^T; at the end the same memory holds the warps' partial results
    const size_t stages = (size_t)WARPS * ((size_t)STAGES * 2 * (PAGE / WARPS) * (D + 8) + NH * (PAGE / WARPS + 8)) * 2;
    const size_t merge = sizeof(float) * ((size_t)WARPS * D * NH + 2 * WARPS * NH);
    const size_t smem = stages > merge ? stages : merge;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<KS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("decode_attention: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(decode_attention_kernel<KS, STAGES>, grid, THREADS, smem, stream, q, ldq, positions, seq_of_token, block_table, max_blocks,
                k_pages, v_pages, n_pages, out, ldo, part_o, part_ml, n_splits, H, Hkv, heads_per_cta, n_chunks, scale, window, newest, status);
    return 0;
}
}  // namespace

// max_new_tokens: the most tokens one request brings in this step (1 when decoding).  Pages that
// lie wholly before a token's last max_new_tokens positions are fetched while earlier kernels
// of the stream may still be writing this step's keys and values.
// Scratch the caller provides when n_splits > 1:
//   part_o  float32 [n_tokens, H, n_splits, D],  part_ml float32 [n_tokens, H, n_splits, 2]
LGML_API long long lgml_decode_attention_scratch_floats(int n_tokens, int H, int D, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * H * n_splits * (D + 2);
}

LGML_API int lgml_decode_attention(const void *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
                                   int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, void *out,
                                   int ldo, float *scratch, int n_splits, int n_tokens, int H, int Hkv, int D, float scale,
                                   int window, int max_new_tokens, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "decode_attention: bad sizes");
    LGML_REQUIRE(page_size == PAGE, "decode_attention: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0, "decode_attention: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D >= 16 && D <= MAX_D && D % 16 == 0, "decode_attention: head_dim %d must be a multiple of 16 up to %d", D, MAX_D);
    LGML_REQUIRE(n_splits >= 1 && n_splits <= MAX_SPLITS, "decode_attention: %d key ranges (1 to %d)", n_splits, MAX_SPLITS);
    LGML_REQUIRE(n_splits == 1 || scratch != nullptr, "decode_attention: %d splits need scratch memory", n_splits);
    LGML_REQUIRE(max_new_tokens >= 1, "decode_attention: max_new_tokens (the most tokens a request brings in this step) must be at least 1");
    {
        static int early = -1;
        if (early < 0) {
            const char *e = getenv("LGML_ATTN_EARLY");
            early = (e != nullptr && e[0] == '0') ? 0 : 1;
        }
        if (!early) max_new_tokens = 1 << 28;     // no page counts as old: every copy waits for the kernels ahead
    }
    LGML_REQUIRE(((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0, "decode_attention: the cache must be 16-byte aligned");
    if (n_tokens == 0) return 0;
    const int group = H / Hkv;
    const int n_chunks = (group + NH - 1) / NH;
    const int heads_per_cta = (group + n_chunks - 1) / n_chunks;   // 1..8 query heads per CTA
    LGML_REQUIRE((long long)Hkv * n_chunks <= 65535, "decode_attention: too many heads");
    LGML_REQUIRE(ldq % 2 == 0 && ((uintptr_t)q & 3) == 0, "decode_attention: q must be 4-byte aligned with an even row stride");
    dim3 grid(n_tokens, Hkv * n_chunks, n_splits);
    float *part_o = scratch;
    float2 *part_ml = reinterpret_cast<float2 *>(scratch + (size_t)n_tokens * H * n_splits * D);
    const __nv_bfloat16 *qq = (const __nv_bfloat16 *)q, *kk = (const __nv_bfloat16 *)k_pages, *vv = (const __nv_bfloat16 *)v_pages;
    __nv_bfloat16 *oo = (__nv_bfloat16 *)out;
    int lrc = 0;
#define LGML_ARGS grid, qq, ldq, positions, seq_of_token, block_table, max_blocks, kk, vv, n_pages, oo, ldo, part_o, part_ml, n_splits, H, Hkv, \
                  heads_per_cta, n_chunks, scale, window, max_new_tokens, status, stream
#define LGML_CASE3(KK) case KK: lrc = launch_ks<KK, 3>(LGML_ARGS); break;
#define LGML_CASE2(KK) case KK: lrc = launch_ks<KK, 2>(LGML_ARGS); break;
    switch (D / 16) {
        LGML_CASE3(1) LGML_CASE3(2) LGML_CASE3(3) LGML_CASE3(4) LGML_CASE3(5) LGML_CASE3(6) LGML_CASE3(7) LGML_CASE3(8)
        LGML_CASE2(9) LGML_CASE2(10) LGML_CASE2(11) LGML_CASE2(12) LGML_CASE2(13) LGML_CASE2(14) LGML_CASE2(15) LGML_CASE2(16)
        default: LGML_FAIL("decode_attention: head_dim %d not handled", D);
    }
#undef LGML_CASE3
#undef LGML_CASE2
#undef LGML_ARGS
    if (lrc) return lrc;
    int rc = lgml_launch_status("decode_attention");
    if (rc) return rc;
    if (n_splits > 1) {
        dim3 cgrid(n_tokens, H);
        lgml_launch(decode_combine_kernel, cgrid, D >= 128 ? 128 : 64, 0, stream, part_o, part_ml, oo, ldo, n_splits, H, D);
        rc = lgml_launch_status("decode_combine");
    }
    return rc;
}
