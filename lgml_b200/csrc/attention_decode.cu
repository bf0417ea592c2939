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
// A page of one KV head is contiguous in the cache ([page][kv head][64][D]), so one thread
// brings it into shared memory with a bulk asynchronous copy (cp.async.bulk, completion on an
// mbarrier); two stages are kept in flight so the copy of the next pages overlaps the math
// of this one.  Per page: (1) scores, 8 lanes per key, each lane 16-byte chunks of the row,
// reduced by shuffles; (2) online softmax per head by one warp; (3) values, threads own 8
// output dimensions and walk the keys.  Softmax, sums and the output accumulators are float32
// (lua/lgml/transformer.lua:1805-1816 for the formula, :1845 for the scale).  Waits on the
// mbarriers are bounded; a wait that runs out sets `status` and the CTA winds down.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_decode)

namespace {
constexpr int PAGE = 64;
constexpr int THREADS = 256;
constexpr int KEYS_PER_WARP = PAGE / (THREADS / 32);   // 8
constexpr int KK = KEYS_PER_WARP / 4;                  // groups of 4 keys a warp walks per page
constexpr int MAX_D = 256;
constexpr uint32_t SPIN_LIMIT = 4u << 20;
constexpr int STATUS_TIMEOUT = 11;

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *status) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(status, STATUS_TIMEOUT);
    return false;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

template <int G, int STAGES>
__global__ void __launch_bounds__(THREADS, 2) decode_attention_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, __nv_bfloat16 *__restrict__ out, int ldo,
    float *__restrict__ part_o, float2 *__restrict__ part_ml, int n_splits, int H, int Hkv, int D, int n_chunks,
    float scale, int window, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // [STAGES][K page | V page] bf16, then the float arrays
    const int page_bytes = PAGE * D * 2;
    uint8_t *kv_s = smem_raw;
    const int n_chunk_ = D / 8;
    const size_t red_bytes = sizeof(float) * (size_t)min(THREADS / n_chunk_, PAGE) * G * D;
    const size_t stage_bytes = (size_t)STAGES * 2 * page_bytes;
    float *qs = reinterpret_cast<float *>(smem_raw + (stage_bytes > red_bytes ? stage_bytes : red_bytes));   // [G][D]
    float *S = qs + G * D;                  // [PAGE][G] scores, then probabilities
    float *m_s = S + PAGE * G;              // [G]
    float *l_s = m_s + G;                   // [G]
    float *corr_s = l_s + G;                // [G]
    float *red = reinterpret_cast<float *>(kv_s);   // [key groups][G][D] for the final sum: the page stages are free by then
    __shared__ uint64_t full_bar[STAGES];
    __shared__ int stage_ok[STAGES];   // whether the stage holds a page (the table had one)

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
    const int n_iter = max(pe - pb, 0);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_bar[s])), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // queries to shared memory as float32, pre-multiplied by the scale
    for (int i = tid; i < G * D; i += THREADS) {
        const int g = i / D, d = i - g * D;
        qs[i] = g < g_count ? to_f32(q[(size_t)t * ldq + (size_t)(h0 + g) * D + d]) * scale : 0.f;
    }
    if (tid < G) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.f;
    }
    __syncthreads();

    // Issue the copy of the page of iteration `it` into stage it % STAGES: only the rows the
    // query can see (rows 0 .. last valid key); a page the table does not hold is skipped.
    auto issue = [&](int it, int page) {
        const int pg = pb + it;
        uint64_t *bar = &full_bar[it % STAGES];
        if (page < 0 || page >= n_pages) {
            atomicExch(status, 3);
            stage_ok[it % STAGES] = 0;
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
            return;
        }
        stage_ok[it % STAGES] = 1;
        const int k_end = min(pos - pg * PAGE + 1, PAGE);
        const uint32_t bytes = (uint32_t)k_end * D * 2;
        const size_t off = ((size_t)page * Hkv + kvh) * PAGE * D;
        uint8_t *dst = kv_s + (size_t)(it % STAGES) * 2 * page_bytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(2 * bytes) : "memory");
        bulk_load(dst, k_pages + off, bytes, bar);
        bulk_load(dst + page_bytes, v_pages + off, bytes, bar);
    };
    if (tid == 0) {
        int first[STAGES];
#pragma unroll
        for (int it = 0; it < STAGES; ++it) first[it] = it < n_iter ? table[pb + it] : -1;   // the loads overlap
#pragma unroll
        for (int it = 0; it < STAGES; ++it)
            if (it < n_iter) issue(it, first[it]);
    }

    const int n_chunk = D / 8;                         // 16-byte chunks per row
    // value phase: thread = (key group, chunk of 8 dims)
    const int KG = min(THREADS / n_chunk, PAGE);
    const bool pv_active = tid < KG * n_chunk;
    const int kgroup = tid / n_chunk, vchunk = tid - kgroup * n_chunk;
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
    // score phase: 8 lanes per key, 4 keys per warp at a time
    const int sub = lane & 7, key_in_warp = lane >> 3;
    bool alive = true;

    for (int it = 0; it < n_iter; ++it) {
        const int pg = pb + it;
        // the table entry of the page STAGES iterations ahead: read now, used at the end of this iteration
        int page_ahead = -1;
        if (tid == 0 && it + STAGES < n_iter) page_ahead = table[pg + STAGES];
        if (alive && !mbar_wait(&full_bar[it % STAGES], (it / STAGES) & 1, status)) alive = false;
        const bool have = stage_ok[it % STAGES] != 0;
        const int k_begin = max(lo - pg * PAGE, 0), k_end = min(pos - pg * PAGE + 1, PAGE);
        const uint8_t *kp = kv_s + (size_t)(it % STAGES) * 2 * page_bytes;
        const uint8_t *vp = kp + page_bytes;

        // ---- (1) scores: warp w takes keys 8w .. 8w+7; lane = (key_in_warp, sub): four keys at a
        // time, 8 lanes per key, lane `sub` owning the 16-byte chunks sub, sub + 8, ... of the row.
        // The queries of a chunk are held in registers while the keys of the warp go by.
        {
            const uint4 *rows4[KK];
            bool key_ok[KK];
#pragma unroll
            for (int kk = 0; kk < KK; ++kk) {
                const int key = warp * KEYS_PER_WARP + kk * 4 + key_in_warp;
                key_ok[kk] = have && alive && key >= k_begin && key < k_end;
                rows4[kk] = reinterpret_cast<const uint4 *>(kp + (size_t)key * D * 2);
            }
            constexpr int GB = G < 4 ? G : 4;           // query heads held in registers at a time
            float s[KK][G];
#pragma unroll
            for (int kk = 0; kk < KK; ++kk)
#pragma unroll
                for (int g = 0; g < G; ++g) s[kk][g] = 0.f;
            for (int c = sub; c < n_chunk; c += 8) {
#pragma unroll
                for (int g0 = 0; g0 < G; g0 += GB) {
                    float qr[GB][8];
#pragma unroll
                    for (int g = 0; g < GB; ++g) {
                        if (g0 + g < G) {
                            const float4 lo4 = *reinterpret_cast<const float4 *>(qs + (size_t)(g0 + g) * D + c * 8);
                            const float4 hi4 = *reinterpret_cast<const float4 *>(qs + (size_t)(g0 + g) * D + c * 8 + 4);
                            qr[g][0] = lo4.x; qr[g][1] = lo4.y; qr[g][2] = lo4.z; qr[g][3] = lo4.w;
                            qr[g][4] = hi4.x; qr[g][5] = hi4.y; qr[g][6] = hi4.z; qr[g][7] = hi4.w;
                        }
                    }
#pragma unroll
                    for (int kk = 0; kk < KK; ++kk) {
                        if (key_ok[kk]) {
                            const uint4 kv4 = rows4[kk][c];
                            const uint32_t w[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
#pragma unroll
                            for (int g = 0; g < GB; ++g) {
                                if (g0 + g < G) {
                                    float a = s[kk][g0 + g];
#pragma unroll
                                    for (int e = 0; e < 4; ++e) a = fmaf(qr[g][2 * e], bf16_lo(w[e]), fmaf(qr[g][2 * e + 1], bf16_hi(w[e]), a));
                                    s[kk][g0 + g] = a;
                                }
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float v = s[kk][g];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    s[kk][g] = v;
                }
                if (sub == 0) {
                    const int key = warp * KEYS_PER_WARP + kk * 4 + key_in_warp;
#pragma unroll
                    for (int g = 0; g < G; ++g) S[key * G + g] = key_ok[kk] ? s[kk][g] : -INFINITY;
                }
            }
        }
        __syncthreads();

        // ---- (2) online softmax, one warp per head ---------------------------------------------
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

        // ---- (3) values --------------------------------------------------------------------------
        if (pv_active) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float c = corr_s[g];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] *= c;
            }
            if (have && alive) {
                for (int key = k_begin + kgroup; key < k_end; key += KG) {
                    const uint4 vv = *reinterpret_cast<const uint4 *>(vp + ((size_t)key * D + vchunk * 8) * 2);
                    const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
                    const float *p = S + key * G;
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float pg_ = p[g];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc[g][2 * e] = fmaf(pg_, bf16_lo(w[e]), acc[g][2 * e]);
                            acc[g][2 * e + 1] = fmaf(pg_, bf16_hi(w[e]), acc[g][2 * e + 1]);
                        }
                    }
                }
            }
        }
        __syncthreads();
        // the stage is free: bring in the page two iterations ahead
        if (tid == 0 && alive && it + STAGES < n_iter) issue(it + STAGES, page_ahead);
    }
    // If a wait ran out, copies may still be in flight: give them a bounded time to land
    // before the shared memory can be handed to another CTA.
    if (!alive && tid == 0) {
        for (int it = max(n_iter - STAGES, 0); it < n_iter; ++it)
            for (uint32_t spin = 0; spin < SPIN_LIMIT && !mbar_try_wait(&full_bar[it % STAGES], (it / STAGES) & 1); ++spin) {
            }
    }

    // ---- sum over key groups, then write ------------------------------------------------------
    if (pv_active) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) red[((size_t)kgroup * G + g) * D + vchunk * 8 + e] = acc[g][e];
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
    pdl_trigger();
    pdl_wait();
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

size_t smem_bytes(int G, int D, int STAGES) {
    const int n_chunk = D / 8;
    int kg = THREADS / n_chunk;
    if (kg > PAGE) kg = PAGE;
    size_t stages = (size_t)STAGES * 2 * PAGE * D * 2, red = sizeof(float) * (size_t)kg * G * D;
    return (stages > red ? stages : red) + sizeof(float) * ((size_t)D * G + (size_t)PAGE * G + 3 * G);
}

template <int G, int STAGES>
int launch_stages(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
           int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo,
           float *part_o, float2 *part_ml, int n_splits, int H, int Hkv, int D, int n_chunks, float scale, int window,
           int *status, cudaStream_t stream) {
    const size_t smem = smem_bytes(G, D, STAGES);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<G, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("decode_attention: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(decode_attention_kernel<G, STAGES>, grid, THREADS, smem, stream, q, ldq, positions, seq_of_token, block_table, max_blocks, k_pages,
                                                               v_pages, n_pages, out, ldo, part_o, part_ml, n_splits, H, Hkv, D,
                                                               n_chunks, scale, window, status);
    return 0;
}

// Three stages while a page of K and V (2 x 64 x D bfloat16) is at most 32 KB, else two.
template <int G>
int launch(dim3 grid, const __nv_bfloat16 *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
           int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, __nv_bfloat16 *out, int ldo,
           float *part_o, float2 *part_ml, int n_splits, int H, int Hkv, int D, int n_chunks, float scale, int window,
           int *status, cudaStream_t stream) {
    if (D <= 128)
        return launch_stages<G, 3>(grid, q, ldq, positions, seq_of_token, block_table, max_blocks, k_pages, v_pages, n_pages, out, ldo,
                                   part_o, part_ml, n_splits, H, Hkv, D, n_chunks, scale, window, status, stream);
    return launch_stages<G, 2>(grid, q, ldq, positions, seq_of_token, block_table, max_blocks, k_pages, v_pages, n_pages, out, ldo,
                               part_o, part_ml, n_splits, H, Hkv, D, n_chunks, scale, window, status, stream);
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
    LGML_REQUIRE(((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0, "decode_attention: the cache must be 16-byte aligned");
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
    int lrc = 0;
#define LGML_CASE(GG)                                                                                                             \
    case GG:                                                                                                                      \
        lrc = launch<GG>(grid, qq, ldq, positions, seq_of_token, block_table, max_blocks, kk, vv, n_pages, oo, ldo, part_o, part_ml, \
                         n_splits, H, Hkv, D, n_chunks, scale, window, status, stream);                                           \
        break;
    switch (G) {
        LGML_CASE(1) LGML_CASE(2) LGML_CASE(3) LGML_CASE(4) LGML_CASE(5) LGML_CASE(6) LGML_CASE(7) LGML_CASE(8)
        default: LGML_FAIL("decode_attention: group of %d heads not handled", G);
    }
#undef LGML_CASE
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
