// Paged attention, general form: any number of query tokens per request (a prompt, a
// portion of one, or one decoded token), keys and values read from the paged cache through
// the request's block table, causal over the request's own cells, with an optional window.
// One block per (token, head); the result of a (token, head) depends only on that token's
// position and its request's cells, in a fixed order, so it is the same however the tokens
// were cut into steps and whatever else is in the batch.  It is the kernel of the 32-bit
// path and the plain device twin of the faster bfloat16 kernels.
//
// softmax over keys of (q . k) * scale with keys at positions <= the query's
// (lua/lgml/transformer.lua:1805-1816, src/lgml.c:2083-2118, mask :2863-2865); head h
// reads KV head h / (H / Hkv).  Scores, the running maximum and the sums are float32.  With
// softcap > 0 a score s becomes softcap * tanh(s / softcap) before the softmax (the reference's
// hp.softcap for other families, lua/lgml/transformer.lua:2097-2102; Llama has none).
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_ref)

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_ref_kernel(
    const T *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const T *__restrict__ k_pages, const T *__restrict__ v_pages,
    int n_pages, int page_size, T *__restrict__ out, int ldo, int H, int Hkv, int D, float scale, int window,
    float softcap, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float qs[MAX_D];
    __shared__ float acc_w[WARPS][MAX_D];
    __shared__ float m_w[WARPS], l_w[WARPS];
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (H / Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int *table = block_table + (size_t)seq * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = to_f32(act_load(q + (size_t)t * ldq + (size_t)h * D + d));
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

    for (int j = lo + warp; j <= pos; j += WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? table[blk] : -1;
        if (page < 0 || page >= n_pages) {  // a cell the table does not hold: flag it, skip the key
            if (lane == 0) atomicExch(status, 3);
            continue;
        }
        const size_t cell = (((size_t)page * Hkv + g) * page_size + (size_t)(j % page_size)) * D;
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) dot = fmaf(qs[d], to_f32(act_load(k_pages + cell + d)), dot);
        float s = warp_sum(dot) * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);   // a cap on the scores (off for Llama)
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) acc[i] = acc[i] * corr + p * to_f32(act_load(v_pages + cell + d));
        }
        m = m_new;
    }
    if (lane == 0) {
        m_w[warp] = m;
        l_w[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc_w[warp][d] = acc[i];
    }
    __syncthreads();
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, m_w[w]);
    float lsum = 0.f;
    float f[WARPS];
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (m_w[w] == -INFINITY) ? 0.f : expf(m_w[w] - mm);
        lsum += l_w[w] * f[w];
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; ++w) o += acc_w[w][d] * f[w];
        out[(size_t)t * ldo + (size_t)h * D + d] = from_f32<T>(lsum > 0.f ? o / lsum : 0.f);
    }
}
}  // namespace

LGML_API int lgml_paged_attention_ref(const void *q, int dtype, int ldq, const int *positions, const int *seq_of_token,
                                      const int *block_table, int max_blocks, const void *k_pages, const void *v_pages,
                                      int n_pages, int page_size, void *out, int ldo, int n_tokens, int H, int Hkv, int D,
                                      float scale, int window, float softcap, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && page_size > 0 && max_blocks > 0, "paged_attention_ref: bad sizes");
    LGML_REQUIRE(H % Hkv == 0, "paged_attention_ref: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D <= MAX_D, "paged_attention_ref: head_dim %d is over %d", D, MAX_D);
    LGML_REQUIRE(H <= 65535, "paged_attention_ref: too many heads");
    LGML_REQUIRE(window >= 0, "paged_attention_ref: bad window");
    LGML_REQUIRE(softcap >= 0.f, "paged_attention_ref: a score cap must be positive (0 = none)");
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, H);
    if (dtype == LGML_F32)
        lgml_launch(paged_attention_ref_kernel<float>, grid, WARPS * 32, 0, stream, 
            (const float *)q, ldq, positions, seq_of_token, block_table, max_blocks, (const float *)k_pages, (const float *)v_pages,
            n_pages, page_size, (float *)out, ldo, H, Hkv, D, scale, window, softcap, status);
    else if (dtype == LGML_BF16)
        lgml_launch(paged_attention_ref_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, stream, 
            (const __nv_bfloat16 *)q, ldq, positions, seq_of_token, block_table, max_blocks, (const __nv_bfloat16 *)k_pages,
            (const __nv_bfloat16 *)v_pages, n_pages, page_size, (__nv_bfloat16 *)out, ldo, H, Hkv, D, scale, window, softcap, status);
    else
        LGML_FAIL("paged_attention_ref: unknown type %d", dtype);
    return lgml_launch_status("paged_attention_ref");
}
