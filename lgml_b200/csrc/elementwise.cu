// Embedding gather, RMSNorm (with the residual add and a row gather fused in), SwiGLU
// activation, bias add and the seeded normal fill.  The residual stream is float32 in
// every mode; norms and the activation compute in float32.
#include <cooperative_groups.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_elementwise)

// ---------------------------------------------------------------------------------------
// x[t, :] = table[ids[t], :]            (lua/lgml/transformer.lua:2303: get_rows, no scale)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_rows_kernel(const TW *__restrict__ table, const int *__restrict__ ids,
                                  float *__restrict__ out, int width, int vocab, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;           // the host checks ids first; never read out of the table
    if (!ok && threadIdx.x == 0 && blockIdx.y == 0) atomicExch(status, 1);
    const TW *row = table + (size_t)(ok ? id : 0) * width;
    const int i0 = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (i0 + j < width) out[(size_t)t * width + i0 + j] = ok ? to_f32(row[i0 + j]) : 0.f;
}

LGML_API int lgml_embed_rows(const void *table, int table_dtype, const int *ids, float *out, int n_tokens,
                             int width, int vocab, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && width > 0 && vocab > 0, "embed_rows: bad sizes");
    if (n_tokens == 0) return 0;
    const int threads = 128;
    dim3 grid(n_tokens, (width + threads * 4 - 1) / (threads * 4));
    if (table_dtype == LGML_F32)
        lgml_launch(embed_rows_kernel<float>, grid, threads, 0, stream, (const float *)table, ids, out, width, vocab, status);
    else if (table_dtype == LGML_BF16)
        lgml_launch(embed_rows_kernel<__nv_bfloat16>, grid, threads, 0, stream, (const __nv_bfloat16 *)table, ids, out, width, vocab, status);
    else
        LGML_FAIL("embed_rows: unknown table type %d", table_dtype);
    return lgml_launch_status("embed_rows");
}

// ---------------------------------------------------------------------------------------
// RMSNorm: y = x / sqrt(mean(x^2) + eps) * w   (src/lgml.c:1626-1633 + the multiply at
// lua/lgml/transformer.lua:1760).  Options, all in one pass over the row:
//   delta != null : x[row] += delta[row] first, and the sum is written back (the residual add)
//   rows  != null : output row r reads x[rows[r]] (the logits' row selection, :2349-2350);
//                   delta is then added for the gathered rows only and x is not written.
// One block per output row; the mean square is summed in a fixed order.
// ---------------------------------------------------------------------------------------
// A row is spread over a thread-block cluster of CS CTAs (CS = 1 for narrow rows): with few
// rows (decoding) one CTA per row would leave the row's bytes to a single SM's memory path.
// Each CTA sums the squares of its slice; the slices' sums are exchanged through distributed
// shared memory and added in rank order.
template <typename TD, typename TO>
__global__ void rmsnorm_kernel(float *__restrict__ x, const TD *__restrict__ delta, int n_parts, long long part_stride,
                               const float *__restrict__ delta_bias, const float *__restrict__ weight,
                               const int *__restrict__ rows, TO *__restrict__ out, int width, float eps, int cs,
                               int clustered) {
    pdl_trigger();
    pdl_wait();
    namespace cg = cooperative_groups;
    __shared__ float red[32];
    __shared__ float slice_ss;
    constexpr int PER = 4;            // elements a thread keeps in registers per round
    // A row is cut into cs slices whose sums of squares are added in slice order.  With few rows
    // the slices run on the CTAs of a cluster; with many rows one CTA walks the slices itself.
    // The arithmetic, and so the result, is the same either way.
    const int r = clustered ? blockIdx.x / cs : blockIdx.x;
    const int rank0 = clustered ? blockIdx.x - r * cs : 0, rank1 = clustered ? rank0 + 1 : cs;
    const int per_cta = ((width + cs - 1) / cs + 3) & ~3;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float *xr = x + src * width;
    const TD *dr = delta ? delta + src * width : nullptr;
    float total = 0.f;
    for (int rank = rank0; rank < rank1; ++rank) {
    const int c0 = rank * per_cta, c1 = min(width, c0 + per_cta);
    float ss = 0.f;
    for (int base = c0; base < c1; base += PER * blockDim.x) {
        // all loads of this round first, so that they are in flight together
        float v[PER], d[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = base + j * blockDim.x + threadIdx.x;
            v[j] = i < c1 ? xr[i] : 0.f;
            d[j] = (dr && i < c1) ? to_f32(act_load(dr + i)) : 0.f;
        }
        if (dr) {
            // the parts are the partial sums of a matrix product cut along K: four are fetched
            // together (their loads overlap), then added in order
            int p = 1;
            for (; p + 4 <= n_parts; p += 4) {
                float e[4][PER];
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                    for (int j = 0; j < PER; ++j) {
                        const int i = base + j * blockDim.x + threadIdx.x;
                        e[q][j] = i < c1 ? to_f32(act_load(dr + (size_t)(p + q) * part_stride + i)) : 0.f;
                    }
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                    for (int j = 0; j < PER; ++j) d[j] += e[q][j];
            }
            for (; p < n_parts; ++p) {
                float e[PER];
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int i = base + j * blockDim.x + threadIdx.x;
                    e[j] = i < c1 ? to_f32(act_load(dr + (size_t)p * part_stride + i)) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < PER; ++j) d[j] += e[j];
            }
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int i = base + j * blockDim.x + threadIdx.x;
                if (i < c1) {
                    if (delta_bias) d[j] += delta_bias[i];
                    v[j] += d[j];
                    if (!rows) xr[i] = v[j];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) ss = fmaf(v[j], v[j], ss);
    }
    total += block_sum(ss, red);
    }
    if (clustered && cs > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        if (threadIdx.x == 0) slice_ss = total;
        cluster.sync();
        total = 0.f;
        for (int k = 0; k < cs; ++k) total += *cluster.map_shared_rank(&slice_ss, k);
        cluster.sync();               // no CTA leaves while another may still read its slice's sum
    }
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    // second pass: with a delta the row was just written (or, with a row list, is summed again the same way)
    const int c0 = rank0 * per_cta, c1 = min(width, rank1 * per_cta);
    for (int base = c0; base < c1; base += PER * blockDim.x) {
        float v[PER], w[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = base + j * blockDim.x + threadIdx.x;
            w[j] = i < c1 ? weight[i] : 0.f;
            v[j] = i < c1 ? xr[i] : 0.f;
        }
        if (dr && rows) {
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int i = base + j * blockDim.x + threadIdx.x;
                if (i < c1) {
                    float d = to_f32(act_load(dr + i));
                    for (int p = 1; p < n_parts; ++p) d += to_f32(act_load(dr + (size_t)p * part_stride + i));
                    if (delta_bias) d += delta_bias[i];
                    v[j] += d;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = base + j * blockDim.x + threadIdx.x;
            if (i < c1) out[(size_t)r * width + i] = from_f32<TO>(v[j] * inv * w[j]);
        }
    }
}

template <typename TD>
static int rmsnorm_dispatch(float *x, const TD *delta, int n_parts, long long part_stride, const float *delta_bias,
                            const float *weight, const int *rows, void *out, int out_dtype, int n_rows, int width, float eps,
                            cudaStream_t stream) {
    // The cluster and block sizes depend on the width only, so a row's sum is formed in the
    // same order whatever else is in the batch.
    const int cs = width >= 2048 ? 8 : (width >= 1024 ? 4 : 1);
    const int clustered = (cs > 1 && n_rows <= 64) ? 1 : 0;     // many rows fill the GPU without clusters
    const int blocks = clustered ? n_rows * cs : n_rows;
    const int threads = 128;
    cudaError_t e;
    if (out_dtype == LGML_F32)
        e = lgml_launch_cluster(rmsnorm_kernel<TD, float>, blocks, threads, 0, stream, clustered ? cs : 1, x, delta, n_parts, part_stride, delta_bias, weight, rows, (float *)out, width, eps, cs, clustered);
    else
        e = lgml_launch_cluster(rmsnorm_kernel<TD, __nv_bfloat16>, blocks, threads, 0, stream, clustered ? cs : 1, x, delta, n_parts, part_stride, delta_bias, weight, rows, (__nv_bfloat16 *)out, width, eps, cs, clustered);
    (void)e;
    return lgml_launch_status("rmsnorm");
}

// delta: null, or [n_parts][rows of x][width] (part_stride elements between parts) whose parts
// are summed in order, plus delta_bias[width] if given.
LGML_API int lgml_rmsnorm(float *x, const void *delta, int delta_dtype, int n_parts, long long part_stride, const float *delta_bias,
                          const float *weight, const int *rows, void *out, int out_dtype, int n_rows, int width, float eps,
                          cudaStream_t stream) {
    LGML_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm: bad sizes");
    LGML_REQUIRE(out_dtype == LGML_F32 || out_dtype == LGML_BF16, "rmsnorm: unknown output type %d", out_dtype);
    LGML_REQUIRE(delta == nullptr || n_parts >= 1, "rmsnorm: a delta has at least one part");
    if (n_rows == 0) return 0;
    if (delta == nullptr || delta_dtype == LGML_F32)
        return rmsnorm_dispatch<float>(x, (const float *)delta, n_parts, part_stride, delta_bias, weight, rows, out, out_dtype, n_rows, width, eps, stream);
    if (delta_dtype == LGML_BF16)
        return rmsnorm_dispatch<__nv_bfloat16>(x, (const __nv_bfloat16 *)delta, n_parts, part_stride, delta_bias, weight, rows, out, out_dtype, n_rows, width, eps, stream);
    LGML_FAIL("rmsnorm: unknown delta type %d", delta_dtype);
}

// ---------------------------------------------------------------------------------------
// act[t, f] = silu(gate[t, f]) * up[t, f], with gate = gu[t, 0:F] and up = gu[t, F:2F]
// (lua/lgml/transformer.lua:2047-2048; silu(a) = a * sigmoid(a), src/lgml.c:1476-1482)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T *__restrict__ gu, T *__restrict__ act, int n_tokens, int width, int paired) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)n_tokens * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width, f = i - t * width;
        const float g = to_f32(act_load(gu + t * 2 * width + (paired ? 2 * f : f)));
        const float u = to_f32(act_load(gu + t * 2 * width + (paired ? 2 * f + 1 : width + f)));
        const float s = g / (1.0f + expf(-g));
        act[i] = from_f32<T>(s * u);
    }
}

// paired: gate and up of feature f are at columns 2f and 2f + 1; else at f and width + f.
LGML_API int lgml_silu_mul(const void *gu, void *act, int dtype, int n_tokens, int width, int paired, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && width > 0, "silu_mul: bad sizes");
    if (n_tokens == 0) return 0;
    const size_t total = (size_t)n_tokens * width;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == LGML_F32)
        lgml_launch(silu_mul_kernel<float>, blocks, threads, 0, stream, (const float *)gu, (float *)act, n_tokens, width, paired);
    else if (dtype == LGML_BF16)
        lgml_launch(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16 *)gu, (__nv_bfloat16 *)act, n_tokens, width, paired);
    else
        LGML_FAIL("silu_mul: unknown type %d", dtype);
    return lgml_launch_status("silu_mul");
}

// ---------------------------------------------------------------------------------------
// x[t, :] += delta[t, :]   (the residual sum in float32 when no norm follows)
// ---------------------------------------------------------------------------------------
template <typename TD>
__global__ void residual_add_kernel(float *__restrict__ x, const TD *__restrict__ delta, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] += to_f32(act_load(delta + i));
}

LGML_API int lgml_residual_add(float *x, const void *delta, int delta_dtype, long long total, cudaStream_t stream) {
    LGML_REQUIRE(total >= 0, "residual_add: bad size");
    if (total == 0) return 0;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (delta_dtype == LGML_F32)
        lgml_launch(residual_add_kernel<float>, blocks, threads, 0, stream, x, (const float *)delta, (size_t)total);
    else if (delta_dtype == LGML_BF16)
        lgml_launch(residual_add_kernel<__nv_bfloat16>, blocks, threads, 0, stream, x, (const __nv_bfloat16 *)delta, (size_t)total);
    else
        LGML_FAIL("residual_add: unknown type %d", delta_dtype);
    return lgml_launch_status("residual_add");
}

// ---------------------------------------------------------------------------------------
// Seeded normal fill: value i of a tensor = mean + sd * N(0,1) from a counter-based stream
// (splitmix64 of seed and index, then Box-Muller; mischief/lgml fills its test tensors the
// same way, src/lgml.c:3064-3079, :3133-3137).  Used to make full-size random models on
// the device without a host copy.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ULL;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T *__restrict__ out, size_t n, float mean, float sd, uint64_t seed) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t h = splitmix64(seed ^ splitmix64(i));
        const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
        const float u2 = (float)(uint32_t)((h >> 8) & 0xffffff) * (1.0f / 16777216.0f);
        const float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        out[i] = from_f32<T>(mean + sd * z);
    }
}

LGML_API int lgml_fill_normal(void *out, int dtype, long long n, float mean, float sd, unsigned long long seed, cudaStream_t stream) {
    LGML_REQUIRE(n >= 0, "fill_normal: bad size");
    if (n == 0) return 0;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    if (dtype == LGML_F32)
        lgml_launch(fill_normal_kernel<float>, blocks, threads, 0, stream, (float *)out, (size_t)n, mean, sd, seed);
    else if (dtype == LGML_BF16)
        lgml_launch(fill_normal_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16 *)out, (size_t)n, mean, sd, seed);
    else
        LGML_FAIL("fill_normal: unknown type %d", dtype);
    return lgml_launch_status("fill_normal");
}
