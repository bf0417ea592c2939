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
