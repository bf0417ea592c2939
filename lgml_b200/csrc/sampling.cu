// Sampling on the device for the neutral chain: argmax (temperature <= 0) or a draw from
// softmax(logits / T) by inverse CDF with a uniform number the host's seeded generator
// supplies.  Same arithmetic as mischief/lgml's sampler: ties go to the lowest index
// (src/sample.c:913-926); logits are divided by T in float32 (:958-960); weights are
// expf(l - max) in float32, their sum and the running sum are float64, the target is
// sum * u, and the first candidate in id order whose running sum reaches it wins
// (draw, :855-877).
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_sampling)

namespace {
constexpr int THREADS = 1024;

struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {  // larger value, then lower index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ Best block_argmax(const float *row, int V, Best *smem) {
    Best best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = act_load(row + i);
        if (v > best.v || (v == best.v && i < best.i)) best = Best{v, i};  // NaN never wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) smem[warp] = best;
    __syncthreads();
    Best total = smem[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) total = better(total, smem[w]);
    if (total.i == 0x7fffffff) total.i = 0;  // a row of NaN or -inf: index 0, as a serial scan from l[0] gives
    return total;
}

__global__ void __launch_bounds__(THREADS) sample_rows_kernel(const float *__restrict__ logits, int ld, int V,
                                                              const float *__restrict__ temperature,
                                                              const double *__restrict__ uniform, int *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ Best best_s[32];
    __shared__ double part[THREADS];
    const int r = blockIdx.x;
    const float *row = logits + (size_t)r * ld;
    const float T = temperature ? temperature[r] : 0.f;
    const Best top = block_argmax(row, V, best_s);
    if (!(T > 0.f)) {
        if (threadIdx.x == 0) out[r] = top.i;
        return;
    }
    const float m = top.v / T;  // the maximum of l / T (T > 0 keeps the order)
    const int chunk = (V + THREADS - 1) / THREADS;
    const int b = threadIdx.x * chunk, e = min(V, b + chunk);
    double s = 0.0;
    for (int i = b; i < e; ++i) s += (double)expf(act_load(row + i) / T - m);
    part[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double sum = 0.0;
        for (int c = 0; c < THREADS; ++c) sum += part[c];
        const double tgt = sum * uniform[r];
        double run = 0.0;
        int c = 0, last_nonzero = 0;
        for (; c < THREADS; ++c) {
            if (part[c] > 0.0) last_nonzero = c;
            if (part[c] > 0.0 && run + part[c] >= tgt) break;
            run += part[c];
        }
        if (c == THREADS) {  // rounding left the target just above the total: the last weight wins
            c = last_nonzero;
            run = 0.0;
            for (int k = 0; k < c; ++k) run += part[k];
        }
        // walk the chunk serially (at most ceil(V / 1024) weights)
        const int cb = c * chunk, ce = min(V, cb + chunk);
        int pick = cb, last = -1;
        bool found = false;
        for (int i = cb; i < ce; ++i) {
            const float w = expf(act_load(row + i) / T - m);
            if (w <= 0.f) continue;
            run += (double)w;
            last = i;
            if (run >= tgt) {
                pick = i;
                found = true;
                break;
            }
        }
        if (!found) pick = last >= 0 ? last : top.i;
        out[r] = pick;
    }
}

// argmax in two passes so that a few rows still use the whole GPU: each row is cut into
// AM_CHUNKS ranges, one block finds the best of a range, then one warp picks among the ranges.
constexpr int AM_CHUNKS = 32;
constexpr int AM_THREADS = 256;

__global__ void __launch_bounds__(AM_THREADS) argmax_partial_kernel(const float *__restrict__ logits, int ld, int V,
                                                                    float *__restrict__ part_v, int *__restrict__ part_i) {
    pdl_trigger();
    pdl_wait();
    __shared__ Best best_s[32];
    const int r = blockIdx.x, c = blockIdx.y;
    const int per = (V + AM_CHUNKS - 1) / AM_CHUNKS;
    const int b = c * per, e = min(V, b + per);
    const float *row = logits + (size_t)r * ld;
    Best best{-INFINITY, 0x7fffffff};
#pragma unroll 4
    for (int i = b + threadIdx.x; i < e; i += AM_THREADS) {
        const float v = act_load(row + i);
        if (v > best.v || (v == best.v && i < best.i)) best = Best{v, i};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) best_s[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        Best total = best_s[0];
        for (int w = 1; w < AM_THREADS / 32; ++w) total = better(total, best_s[w]);
        part_v[r * AM_CHUNKS + c] = total.v;
        part_i[r * AM_CHUNKS + c] = total.i;
    }
}

__global__ void argmax_final_kernel(const float *__restrict__ part_v, const int *__restrict__ part_i, int *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, lane = threadIdx.x;
    Best best{act_load(part_v + r * AM_CHUNKS + lane), (int)act_load(reinterpret_cast<const unsigned int *>(part_i) + r * AM_CHUNKS + lane)};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;   // a row of NaN or -inf: index 0
}

// ---------------------------------------------------------------------------------------------
// The k best candidates of every row, ordered by (logit descending, id ascending): the first
// step of the sampler's chain after bias and penalties (top_k, src/sample.c:769-790; the order of
// sorted candidates :680-688).  The rest of the chain works on these k values, so with top_k on
// the host needs k pairs per row, not the row.
// One block per row.  A candidate's key is 64 bits: the logit's bits made monotonic, then the
// complement of the id, so keys are distinct and a larger key is a better candidate.  The k-th
// largest key is found by radix selection, 11 bits a pass from the top, stopping as soon as
// the keys that still tie on the bits seen fit shared memory, where they are sorted; then the
// keys at or above the k-th are gathered and sorted.  NaN sorts last.
// ---------------------------------------------------------------------------------------------
constexpr int TK_THREADS = 1024;
constexpr int TK_BITS = 11, TK_BINS = 1 << TK_BITS;
constexpr int TK_CAP = 1024;          // keys sorted in shared memory at once
constexpr int TK_MAX_K = 128;

__device__ __forceinline__ unsigned long long topk_key(float v, int id) {
    unsigned int u = __float_as_uint(v);
    if (v != v) u = 0u;                                            // NaN: below everything
    else u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);          // monotonic in v
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned int)id);
}

// sort keys[0 .. n) descending; n a power of two up to TK_CAP; all threads of the block call it
__device__ void topk_sort_desc(unsigned long long *keys, int n) {
    for (int size = 2; size <= n; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1)), hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a < b) == desc) {
                    keys[lo] = b;
                    keys[hi] = a;
                }
            }
        }
    __syncthreads();
}

__global__ void __launch_bounds__(TK_THREADS) topk_rows_kernel(const float *__restrict__ logits, int ld, int V, int k, float *__restrict__ out_vals,
                                                               int *__restrict__ out_ids) {
    pdl_trigger();
    pdl_wait();
    __shared__ unsigned int hist[TK_BINS];
    __shared__ unsigned int warp_tot[32];
    __shared__ unsigned long long keys[TK_CAP];
    __shared__ unsigned long long s_prefix, s_threshold;
    __shared__ unsigned int s_need, s_count, s_bin_count;
    const float *row = logits + (size_t)blockIdx.x * ld;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    unsigned long long prefix = 0, mask = 0;       // the bits decided so far and where they are
    unsigned int need = (unsigned int)k;           // how many of the keys that match the prefix are wanted
    int shift = 64 - TK_BITS;
    while (true) {
        const int bits = shift >= 0 ? TK_BITS : TK_BITS + shift;     // the last pass may be narrower
        const int sh = shift >= 0 ? shift : 0;
        const unsigned int digit_mask = (1u << bits) - 1u;
        for (int i = tid; i < TK_BINS; i += TK_THREADS) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < V; i += TK_THREADS) {
            const unsigned long long key = topk_key(act_load(row + i), i);
            if ((key & mask) == prefix) atomicAdd(&hist[(unsigned int)(key >> sh) & digit_mask], 1u);
        }
        __syncthreads();
        // suffix sums over the bins (two bins a thread): S(t) = keys with a digit >= 2t
        const unsigned int h0 = hist[2 * tid], h1 = hist[2 * tid + 1];
        unsigned int suf = h0 + h1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int other = __shfl_down_sync(0xffffffffu, suf, o);
            if (lane + o < 32) suf += other;
        }
        if (lane == 0) warp_tot[warp] = suf;
        __syncthreads();
        unsigned int after = 0;                                       // keys in the warps above this one
        for (int w = warp + 1; w < 32; ++w) after += warp_tot[w];
        const unsigned int s_here = suf + after;                      // digits >= 2 tid
        const unsigned int s_next = s_here - (h0 + h1);               // digits >= 2 tid + 2
        if (s_here >= need && s_next < need) {
            // the k-th key has its digit in this thread's pair of bins
            unsigned int digit, above;
            if (s_next + h1 >= need) {
                digit = 2 * tid + 1;
                above = s_next;
            } else {
                digit = 2 * tid;
                above = s_next + h1;
            }
            s_prefix = prefix | ((unsigned long long)digit << sh);
            s_need = need - above;
            s_bin_count = digit == 2 * (unsigned int)tid + 1 ? h1 : h0;
        }
        __syncthreads();
        prefix = s_prefix;
        mask |= (unsigned long long)digit_mask << sh;
        need = s_need;
        const unsigned int in_bin = s_bin_count;
        __syncthreads();
        if (in_bin <= TK_CAP || sh == 0) break;                       // (at sh == 0 all bits are decided: one key is left)
        shift -= TK_BITS;
    }
    // the keys that match the prefix, sorted: the need-th of them is the k-th key of the row
    if (tid == 0) s_count = 0;
    for (int i = tid; i < TK_CAP; i += TK_THREADS) keys[i] = 0ull;
    __syncthreads();
    for (int i = tid; i < V; i += TK_THREADS) {
        const unsigned long long key = topk_key(act_load(row + i), i);
        if ((key & mask) == prefix) {
            const unsigned int at = atomicAdd(&s_count, 1u);
            if (at < TK_CAP) keys[at] = key;
        }
    }
    __syncthreads();
    int n = 2;
    while (n < (int)min(s_count, (unsigned int)TK_CAP)) n <<= 1;
    topk_sort_desc(keys, n);
    if (tid == 0) s_threshold = keys[need - 1];
    __syncthreads();
    const unsigned long long threshold = s_threshold;
    __syncthreads();
    // gather the k keys at or above the k-th, sort them, write values and ids
    if (tid == 0) s_count = 0;
    for (int i = tid; i < TK_MAX_K; i += TK_THREADS) keys[i] = 0ull;
    __syncthreads();
    for (int i = tid; i < V; i += TK_THREADS) {
        const float v = act_load(row + i);
        const unsigned long long key = topk_key(v, i);
        if (key >= threshold) {
            const unsigned int at = atomicAdd(&s_count, 1u);
            if (at < TK_MAX_K) keys[at] = key;
        }
    }
    __syncthreads();
    topk_sort_desc(keys, TK_MAX_K);
    for (int j = tid; j < k; j += TK_THREADS) {
        const unsigned long long key = keys[j];
        const int id = (int)(0xffffffffu - (unsigned int)(key & 0xffffffffull));
        out_ids[(size_t)blockIdx.x * k + j] = id;
        out_vals[(size_t)blockIdx.x * k + j] = act_load(row + id);
    }
}

// ---------------------------------------------------------------------------------------------
// The first two steps of the sampler's chain, in place on the rows of logits: the logit bias
// (l[id] += b) and then the history penalties over the distinct ids of a request's recent
// tokens (src/sample.c:1051-1053, apply_penalties :652-677): v = l[id]; v = v * repeat if
// v <= 0 else v / repeat; l[id] = v - (count * frequency + presence), every step rounded to
// float32.  One warp per row; the ids within a step are distinct, so its lanes do not collide.
// edits: per row  [n_bias, n_hist, then n_bias x (id, value bits), then n_hist x (id, count)]
// at offset row * stride (int32 words); params: per row (repeat, frequency, presence).
// ---------------------------------------------------------------------------------------------
__global__ void sampler_edits_kernel(float *__restrict__ logits, int ld, int V, const int *__restrict__ edits, int stride,
                                     const float *__restrict__ params) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, lane = threadIdx.x;
    float *row = logits + (size_t)r * ld;
    const int *e = edits + (size_t)r * stride;
    const int n_bias = e[0], n_hist = e[1];
    for (int i = lane; i < n_bias; i += 32) {
        const int id = e[2 + 2 * i];
        if (id >= 0 && id < V) row[id] = __fadd_rn(row[id], __int_as_float(e[3 + 2 * i]));
    }
    __syncwarp();
    const float rep = params[3 * r], freq = params[3 * r + 1], pres = params[3 * r + 2];
    const int *h = e + 2 + 2 * n_bias;
    for (int i = lane; i < n_hist; i += 32) {
        const int id = h[2 * i];
        if (id < 0 || id >= V) continue;
        float v = row[id];
        v = v <= 0.f ? __fmul_rn(v, rep) : __fdiv_rn(v, rep);
        row[id] = __fsub_rn(v, __fadd_rn(__fmul_rn((float)h[2 * i + 1], freq), pres));
    }
}

// ---------------------------------------------------------------------------------------------
// The rest of the chain on the k candidates that top_k left (sorted: logit descending, id
// ascending): top_p, min_p, temperature and the draw, one thread per row, every step in the
// arithmetic of the host sampler (src/sample.c:808-877): top_p keeps the shortest prefix whose
// float32 running sum of exp(l - l0) / total reaches p; min_p keeps logits >= l0 + ln(p);
// the logits are divided by T in float32; the draw takes float32 weights exp(l / T - max),
// sums them in float64 and picks the first candidate whose running sum reaches sum * u.
// params per row: top_p, ln(min_p) (or -inf), T;  uniform per row: u in [0, 1).
// ---------------------------------------------------------------------------------------------
__global__ void sample_candidates_kernel(const float *__restrict__ vals, const int *__restrict__ ids, int k, const float *__restrict__ params,
                                         const double *__restrict__ uniform, int *__restrict__ out, int n_rows) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const float *v = vals + (size_t)r * k;
    const int *id = ids + (size_t)r * k;
    const float top_p = params[3 * r], log_min_p = params[3 * r + 1], T = params[3 * r + 2];
    if (!(T > 0.f)) {             // the argmax: the first candidate (ties went to the lowest id)
        out[r] = __ldcg(id);
        return;
    }
    const float v0 = act_load(v);
    int keep = k;
    if (top_p < 1.0f) {
        float total = 0.f;
        for (int i = 0; i < k; ++i) total = __fadd_rn(total, expf(__fsub_rn(act_load(v + i), v0)));
        float cum = 0.f;
        for (int i = 0; i < k; ++i) {
            cum = __fadd_rn(cum, __fdiv_rn(expf(__fsub_rn(act_load(v + i), v0)), total));
            if (cum >= top_p) {
                keep = i + 1;
                break;
            }
        }
    }
    if (log_min_p > -INFINITY) {
        const float thr = __fadd_rn(v0, log_min_p);
        int n = 0;
        while (n < keep && act_load(v + n) >= thr) ++n;       // sorted: the kept ones are a prefix
        keep = n > 0 ? n : 1;
    }
    const float m = T != 1.0f ? __fdiv_rn(v0, T) : v0;
    double sum = 0.0;
    for (int i = 0; i < keep; ++i) {
        const float l = T != 1.0f ? __fdiv_rn(act_load(v + i), T) : act_load(v + i);
        sum += (double)expf(__fsub_rn(l, m));
    }
    const double tgt = sum * uniform[r];
    double run = 0.0;
    int pick = -1, last = 0;
    for (int i = 0; i < keep; ++i) {
        const float l = T != 1.0f ? __fdiv_rn(act_load(v + i), T) : act_load(v + i);
        const float w = expf(__fsub_rn(l, m));
        if (w <= 0.f) continue;
        run += (double)w;
        last = i;
        if (run >= tgt) {
            pick = i;
            break;
        }
    }
    out[r] = __ldcg(id + (pick >= 0 ? pick : last));
}
}  // namespace

// scratch: n_rows * 32 floats and n_rows * 32 ints (lgml_argmax_scratch_words words in all).
LGML_API long long lgml_argmax_scratch_words(int n_rows) { return 2LL * n_rows * AM_CHUNKS; }

LGML_API int lgml_argmax_rows(const float *logits, int ld, int n_rows, int V, int *out, void *scratch, cudaStream_t stream) {
    LGML_REQUIRE(n_rows >= 0 && V > 0 && ld >= V, "argmax_rows: bad sizes");
    LGML_REQUIRE(scratch != nullptr || n_rows == 0, "argmax_rows: scratch memory is missing");
    if (n_rows == 0) return 0;
    float *part_v = (float *)scratch;
    int *part_i = (int *)scratch + (size_t)n_rows * AM_CHUNKS;
    lgml_launch(argmax_partial_kernel, dim3(n_rows, AM_CHUNKS), AM_THREADS, 0, stream, logits, ld, V, part_v, part_i);
    int rc = lgml_launch_status("argmax_rows");
    if (rc) return rc;
    lgml_launch(argmax_final_kernel, n_rows, 32, 0, stream, (const float *)part_v, (const int *)part_i, out);
    return lgml_launch_status("argmax_rows final");
}

// temperature[r] <= 0 takes the argmax of row r; uniform[r] in [0, 1) is used otherwise.
LGML_API int lgml_sample_rows(const float *logits, int ld, int n_rows, int V, const float *temperature, const double *uniform,
                              int *out, cudaStream_t stream) {
    LGML_REQUIRE(n_rows >= 0 && V > 0 && ld >= V, "sample_rows: bad sizes");
    if (n_rows == 0) return 0;
    lgml_launch(sample_rows_kernel, n_rows, THREADS, 0, stream, logits, ld, V, temperature, uniform, out);
    return lgml_launch_status("sample_rows");
}

// out_vals, out_ids: [n_rows, k], the k best candidates of each row by (logit descending, id
// ascending); 1 <= k <= min(V, 128).
LGML_API int lgml_topk_rows(const float *logits, int ld, int n_rows, int V, int k, float *out_vals, int *out_ids, cudaStream_t stream) {
    LGML_REQUIRE(n_rows >= 0 && V > 0 && ld >= V, "topk_rows: bad sizes");
    LGML_REQUIRE(k >= 1 && k <= TK_MAX_K && k <= V, "topk_rows: k = %d must be between 1 and min(vocabulary %d, %d)", k, V, TK_MAX_K);
    if (n_rows == 0) return 0;
    lgml_launch(topk_rows_kernel, n_rows, TK_THREADS, 0, stream, logits, ld, V, k, out_vals, out_ids);
    return lgml_launch_status("topk_rows");
}

// Bias and history penalties of the sampler's chain, in place (see sampler_edits_kernel for the
// layout of `edits` and `params`).
LGML_API int lgml_sampler_edits(float *logits, int ld, int n_rows, int V, const int *edits, int stride, const float *params,
                                cudaStream_t stream) {
    LGML_REQUIRE(n_rows >= 0 && V > 0 && ld >= V && stride >= 2, "sampler_edits: bad sizes");
    if (n_rows == 0) return 0;
    lgml_launch(sampler_edits_kernel, n_rows, 32, 0, stream, logits, ld, V, edits, stride, params);
    return lgml_launch_status("sampler_edits");
}

// vals, ids: [n_rows, k] from lgml_topk_rows; params float32 [n_rows, 3] = top_p, ln(min_p) or
// -inf, temperature (<= 0: the first candidate); uniform float64 [n_rows]; out int32 [n_rows].
LGML_API int lgml_sample_candidates(const float *vals, const int *ids, int n_rows, int k, const float *params, const double *uniform,
                                    int *out, cudaStream_t stream) {
    LGML_REQUIRE(n_rows >= 0 && k >= 1, "sample_candidates: bad sizes");
    if (n_rows == 0) return 0;
    lgml_launch(sample_candidates_kernel, (n_rows + 31) / 32, 32, 0, stream, vals, ids, k, params, uniform, out, n_rows);
    return lgml_launch_status("sample_candidates");
}
