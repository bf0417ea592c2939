// Paged attention for decoding (and short portions), bfloat16 cache, float32 math.
//
// Every query token is independent: token t of request s at position p attends to the
// cells of s at positions <= p (the last `window` of them if a window is set).  The work of
// one token is cut by KV head and, along the keys, into `n_splits` ranges of whole pages;
// one CTA handles (token, KV head [x chunk of its query heads], split).  The query heads
// that share a KV head (grouped-query attention) are processed together, so each key and
// value is read from HBM once for all of them.  A split leaves an unnormalised partial
// result (running maximum m, sum l, weighted values O) in scratch memory; a second kernel
// merges the splits in a fixed order.  With one split the result is written directly.
//
// Per page of 64 keys a CTA does three phases: (1) scores: two threads per key read the
// key row with 16-byte loads and dot it with all query heads, which sit in shared memory as
// float32; (2) online softmax per head by one warp; (3) values: threads own pairs of output
// dimensions and walk the keys.  Softmax, sums and the output accumulators are float32
// (lua/lgml/transformer.lua:1805-1816 for the formula, :1845 for the scale).
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_decode)

namespace {
constexpr int PAGE = 64;
constexpr int THREADS = 128;
constexpr int MAX_D = 256;

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

template <int G>
__global__ void __launch_bounds__(THREADS) decode_attention_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, __nv_bfloat16 *__restrict__ out, int ldo,
    float *__restrict__ part_o, float2 *__restrict__ part_ml, int n_splits, int H, int Hkv, int D, int n_chunks,
    float scale, int window, int *__restrict__ status) {
    extern __shared__ float smem[];
    float *qs = smem;                       // [D][G]
    float *S = qs + D * G;                  // [PAGE][G] scores, then probabilities
    float *m_s = S + PAGE * G;              // [G]
    float *l_s = m_s + G;                   // [G]
    float *corr_s = l_s + G;                // [G]
    float *red = corr_s + G;                // [KG][G][D] for the final sum over key groups

    const int t = blockIdx.x;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    const int split = blockIdx.z;
    const int group = H / Hkv;
    const int h0 = kvh * group + chunk * G;                       // first query head of this CTA
    const int g_count = min(G, group - chunk * G);                // heads it really has
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

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

    // queries to shared memory as float32, pre-multiplied by the scale
    for (int i = tid; i < D * G; i += THREADS) {
        const int d = i / G, g = i - d * G;
        qs[i] = g < g_count ? to_f32(q[(size_t)t * ldq + (size_t)(h0 + g) * D + d]) * scale : 0.f;
    }
    if (tid < G) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.f;
    }
    const int NPAIR = D / 2;
    const int KG = THREADS / NPAIR > PAGE ? PAGE : THREADS / NPAIR;   // key groups of the value phase
    const bool pv_active = tid < KG * NPAIR;
    const int kgroup = tid / NPAIR, pi = tid - kgroup * NPAIR;
    float acc[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g][0] = acc[g][1] = 0.f;
    __syncthreads();

    const int key_local = tid >> 1, half = tid & 1;
    const int half_d = D / 2;
    const int nvec = half_d / 8;                                   // 16-byte loads per thread per key

    for (int pg = pb; pg < pe; ++pg) {
        const int page = table[pg];
        if (page < 0 || page >= n_pages) {                         // the table does not hold this block: flag, skip
            if (tid == 0) atomicExch(status, 3);
            continue;
        }
        const int k_begin = max(lo - pg * PAGE, 0), k_end = min(pos - pg * PAGE + 1, PAGE);
        const __nv_bfloat16 *kp = k_pages + ((size_t)page * Hkv + kvh) * PAGE * D;
        const __nv_bfloat16 *vp = v_pages + ((size_t)page * Hkv + kvh) * PAGE * D;

        // ---- (1) scores --------------------------------------------------------------------
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
        const bool key_ok = key_local >= k_begin && key_local < k_end;
        if (key_ok) {
            const uint4 *row = reinterpret_cast<const uint4 *>(kp + (size_t)key_local * D + half * half_d);
            const float *qh = qs + (size_t)half * half_d * G;
#pragma unroll 4
            for (int c = 0; c < nvec; ++c) {
                const uint4 kk = row[c];
                const uint32_t w[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float k0 = bf16_lo(w[e]), k1 = bf16_hi(w[e]);
                    const float *q0 = qh + (size_t)(c * 8 + e * 2) * G;
#pragma unroll
                    for (int g = 0; g < G; ++g) s[g] = fmaf(q0[g], k0, s[g]);
#pragma unroll
                    for (int g = 0; g < G; ++g) s[g] = fmaf(q0[G + g], k1, s[g]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
            if (half == 0) S[key_local * G + g] = key_ok ? s[g] : -INFINITY;
        }
        __syncthreads();

        // ---- (2) online softmax, one warp per head -----------------------------------------
        for (int g = warp; g < G; g += THREADS / 32) {
            const float s0 = S[lane * G + g], s1 = S[(lane + 32) * G + g];
            const float mx = warp_max(fmaxf(s0, s1));
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, mx);
            float p0 = 0.f, p1 = 0.f, corr = 1.f;
            if (m_new != -INFINITY) {
                corr = expf(m_old - m_new);
                p0 = expf(s0 - m_new);
                p1 = expf(s1 - m_new);
            }
            const float ls = warp_sum(p0 + p1);
            S[lane * G + g] = p0;
            S[(lane + 32) * G + g] = p1;
            if (lane == 0) {
                m_s[g] = m_new;
                l_s[g] = l_s[g] * corr + ls;
                corr_s[g] = corr;
            }
        }
        __syncthreads();

        // ---- (3) values --------------------------------------------------------------------
        if (pv_active) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float c = corr_s[g];
                acc[g][0] *= c;
                acc[g][1] *= c;
            }
            const uint32_t *vcol = reinterpret_cast<const uint32_t *>(vp) + pi;
#pragma unroll 4
            for (int key = k_begin + kgroup; key < k_end; key += KG) {
                const uint32_t vv = vcol[(size_t)key * NPAIR];
                const float v0 = bf16_lo(vv), v1 = bf16_hi(vv);
                const float *p = S + key * G;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    acc[g][0] = fmaf(p[g], v0, acc[g][0]);
                    acc[g][1] = fmaf(p[g], v1, acc[g][1]);
                }
            }
        }
        __syncthreads();
    }

    // ---- sum over key groups, then write ------------------------------------------------------
    if (pv_active) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            red[((size_t)kgroup * G + g) * D + 2 * pi] = acc[g][0];
            red[((size_t)kgroup * G + g) * D + 2 * pi + 1] = acc[g][1];
        }
    }
    __syncthreads();
    for (int i = tid; i < g_count * D; i += THREADS) {
        const int g = i / D, d = i - g * D;
        float o = 0.f;
        for (int kg = 0; kg < KG; ++kg) o += red[((size_t)kg * G + g) * D + d];
        const int h = h0 + g;
        if (n_splits == 1) {
            const float l = l_s[g];
            out[(size_t)t * ldo + (size_t)h * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            part_o[(((size_t)t * H + h) * n_splits + split) * D + d] = o;
        }
    }
    if (n_splits > 1 && tid < g_count)
        part_ml[((size_t)t * H + h0 + tid) * n_splits + split] = make_float2(m_s[tid], l_s[tid]);
}

// Merge the splits of one (token, head) in split order.
__global__ void decode_combine_kernel(const float *__restrict__ part_o, const float2 *__restrict__ part_ml,
                                      __nv_bfloat16 *__restrict__ out, int ldo, int n_splits, int H, int D) {
    const int t = blockIdx.x, h = blockIdx.y;
    const float2 *ml = part_ml + ((size_t)t * H + h) * n_splits;
    float mm = -INFINITY;
    for (int i = 0; i < n_splits; ++i) mm = fmaxf(mm, ml[i].x);
    float l = 0.f;
    for (int i = 0; i < n_splits; ++i) l += ml[i].x == -INFINITY ? 0.f : ml[i].y * expf(ml[i].x - mm);
    const float *po = part_o + ((size_t)t * H + h) * n_splits * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int i = 0; i < n_splits; ++i)
            if (ml[i].x != -INFINITY) o += po[(size_t)i * D + d] * expf(ml[i].x - mm);
        out[(size_t)t * ldo + (size_t)h * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

size_t smem_bytes(int G, int D) {
    const int npair = D / 2;
    int kg = THREADS / npair;
    if (kg > PAGE) kg = PAGE;
    return sizeof(float) * ((size_t)D * G + (size_t)PAGE * G + 3 * G + (size_t)kg * G * D);
}

template <int G>
int launch(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
           int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo,
           float *part_o, float2 *part_ml, int n_splits, int H, int Hkv, int D, int n_chunks, float scale, int window,
           int *status, cudaStream_t stream) {
    const size_t smem = smem_bytes(G, D);
    if (smem > 48 * 1024) cudaFuncSetAttribute(decode_attention_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    decode_attention_kernel<G><<<grid, THREADS, smem, stream>>>(q, ldq, positions, seq_of_token, block_table, max_blocks, k_pages,
                                                               v_pages, n_pages, out, ldo, part_o, part_ml, n_splits, H, Hkv, D,
                                                               n_chunks, scale, window, status);
    return 0;
}
}  // namespace

// Scratch the caller provides when n_splits > 1:
//   part_o  float32 [n_tokens, H, n_splits, D],  part_ml float32 [n_tokens, H, n_splits, 2]
LGML_API long long lgml_decode_attention_scratch_floats(int n_tokens, int H, int D, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * H * n_splits * (D + 2);
}

LGML_API int lgml_decode_attention(const void *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
                                   int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, void *out,
                                   int ldo, float *scratch, int n_splits, int n_tokens, int H, int Hkv, int D, float scale,
                                   int window, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "decode_attention: bad sizes");
    LGML_REQUIRE(page_size == PAGE, "decode_attention: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0, "decode_attention: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D >= 16 && D <= MAX_D && D % 16 == 0, "decode_attention: head_dim %d must be a multiple of 16 up to %d", D, MAX_D);
    LGML_REQUIRE(n_splits >= 1 && n_splits <= 65535, "decode_attention: bad split count %d", n_splits);
    LGML_REQUIRE(n_splits == 1 || scratch != nullptr, "decode_attention: %d splits need scratch memory", n_splits);
    if (n_tokens == 0) return 0;
    const int group = H / Hkv;
    const int n_chunks = (group + 7) / 8;
    const int G = (group + n_chunks - 1) / n_chunks;   // 1..8 query heads per CTA
    LGML_REQUIRE((long long)Hkv * n_chunks <= 65535, "decode_attention: too many heads");
    dim3 grid(n_tokens, Hkv * n_chunks, n_splits);
    float *part_o = scratch;
    float2 *part_ml = reinterpret_cast<float2 *>(scratch + (size_t)n_tokens * H * n_splits * D);
    const __nv_bfloat16 *qq = (const __nv_bfloat16 *)q, *kk = (const __nv_bfloat16 *)k_pages, *vv = (const __nv_bfloat16 *)v_pages;
    __nv_bfloat16 *oo = (__nv_bfloat16 *)out;
#define LGML_CASE(GG)                                                                                                             \
    case GG:                                                                                                                      \
        launch<GG>(grid, qq, ldq, positions, seq_of_token, block_table, max_blocks, kk, vv, n_pages, oo, ldo, part_o, part_ml,    \
                   n_splits, H, Hkv, D, n_chunks, scale, window, status, stream);                                                 \
        break;
    switch (G) {
        LGML_CASE(1) LGML_CASE(2) LGML_CASE(3) LGML_CASE(4) LGML_CASE(5) LGML_CASE(6) LGML_CASE(7) LGML_CASE(8)
        default: LGML_FAIL("decode_attention: group of %d heads not handled", G);
    }
#undef LGML_CASE
    int rc = lgml_launch_status("decode_attention");
    if (rc) return rc;
    if (n_splits > 1) {
        dim3 cgrid(n_tokens, H);
        decode_combine_kernel<<<cgrid, D >= 128 ? 128 : 64, 0, stream>>>(part_o, part_ml, oo, ldo, n_splits, H, D);
        rc = lgml_launch_status("decode_combine");
    }
    return rc;
}
