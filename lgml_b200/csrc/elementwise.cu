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
//
// One order of arithmetic for every way of launching it, so that a row's result has the same
// bits whatever else is in the batch.  A row is cut into `cs` slices (8 for wide rows, the
// width alone decides).  A slice belongs to a group of 128 threads; in round rd thread g of the
// group holds the four consecutive elements  slice start + 512 rd + 4 g ...+3  (one 16-byte
// access when the row allows it), adds their squares in that order, the group adds its threads'
// sums by warp trees and then the four warps' sums by index, and the slices' sums are added by
// index.  Four ways of launching share this:
//   - few rows (decoding): the slices of a row are the groups of 128 threads of one block (a
//     slice then has at most 1,024 elements); for wider rows they are the CTAs of a thread-block
//     cluster, whose sums cross through distributed shared memory;
//   - many rows (prompts): one block of 128 threads takes all slices of its row one after the
//     other, with every load of the row issued before any is used;
//   - rows too wide for the registers of those two: one block per row that walks the row twice.
// ---------------------------------------------------------------------------------------
namespace rms {
constexpr int PER = 4, GROUP = 128, WARPS = GROUP / 32, MAX_CS = 8;

__device__ __forceinline__ void load_quad(const float *p, int i, int c1, bool vec, float (&o)[PER]) {
    if (vec && i + PER <= c1) {
        const float4 t = act_load(reinterpret_cast<const float4 *>(p + i));
        o[0] = t.x, o[1] = t.y, o[2] = t.z, o[3] = t.w;
    } else {
#pragma unroll
        for (int e = 0; e < PER; ++e) o[e] = i + e < c1 ? act_load(p + i + e) : 0.f;
    }
}
__device__ __forceinline__ void load_quad(const __nv_bfloat16 *p, int i, int c1, bool vec, float (&o)[PER]) {
    if (vec && i + PER <= c1) {
        const float2 raw = act_load(reinterpret_cast<const float2 *>(p + i));       // 8 bytes = 4 bfloat16
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
        o[0] = __bfloat162float(lo.x), o[1] = __bfloat162float(lo.y), o[2] = __bfloat162float(hi.x), o[3] = __bfloat162float(hi.y);
    } else {
#pragma unroll
        for (int e = 0; e < PER; ++e) o[e] = i + e < c1 ? __bfloat162float(act_load(p + i + e)) : 0.f;
    }
}
// weights and biases: not written by any kernel of the stream
__device__ __forceinline__ void load_quad_const(const float *p, int i, int c1, bool vec, float (&o)[PER]) {
    if (vec && i + PER <= c1) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p + i));
        o[0] = t.x, o[1] = t.y, o[2] = t.z, o[3] = t.w;
    } else {
#pragma unroll
        for (int e = 0; e < PER; ++e) o[e] = i + e < c1 ? __ldg(p + i + e) : 0.f;
    }
}
__device__ __forceinline__ void store_quad(float *p, int i, int c1, bool vec, const float (&v)[PER]) {
    if (vec && i + PER <= c1) {
        *reinterpret_cast<float4 *>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
        for (int e = 0; e < PER; ++e)
            if (i + e < c1) p[i + e] = v[e];
    }
}
__device__ __forceinline__ void store_quad(__nv_bfloat16 *p, int i, int c1, bool vec, const float (&v)[PER]) {
    if (vec && i + PER <= c1) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        float2 raw;
        raw.x = *reinterpret_cast<float *>(&lo), raw.y = *reinterpret_cast<float *>(&hi);
        *reinterpret_cast<float2 *>(p + i) = raw;
    } else {
#pragma unroll
        for (int e = 0; e < PER; ++e)
            if (i + e < c1) p[i + e] = __float2bfloat16_rn(v[e]);
    }
}

// Four elements as they lie in memory, for loads that are all issued before any is used: a
// bfloat16 quad then waits in two registers, not four.
template <typename T> struct RawQuad;
template <> struct RawQuad<float> {
    float v[PER];
    __device__ __forceinline__ void load(const float *p, int i, int c1, bool vec) { load_quad(p, i, c1, vec, v); }
    __device__ __forceinline__ void get(float (&o)[PER]) const {
#pragma unroll
        for (int e = 0; e < PER; ++e) o[e] = v[e];
    }
};
template <> struct RawQuad<__nv_bfloat16> {
    __nv_bfloat162 lo, hi;
    __device__ __forceinline__ void load(const __nv_bfloat16 *p, int i, int c1, bool vec) {
        if (vec && i + PER <= c1) {
            const float2 raw = act_load(reinterpret_cast<const float2 *>(p + i));
            lo = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
        } else {
            const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
            lo.x = i < c1 ? act_load(p + i) : z, lo.y = i + 1 < c1 ? act_load(p + i + 1) : z;
            hi.x = i + 2 < c1 ? act_load(p + i + 2) : z, hi.y = i + 3 < c1 ? act_load(p + i + 3) : z;
        }
    }
    __device__ __forceinline__ void get(float (&o)[PER]) const {
        o[0] = __bfloat162float(lo.x), o[1] = __bfloat162float(lo.y), o[2] = __bfloat162float(hi.x), o[3] = __bfloat162float(hi.y);
    }
};

struct Args {
    float *x;
    const void *delta;
    int n_parts;
    long long part_stride;
    const float *delta_bias, *weight;
    const int *rows;
    void *out;
    int width;
    float eps;
    int cs;
    int vec;      // rows, parts and vectors allow 16-byte accesses (8-byte for bfloat16)
};

// d += parts 1 .. n_parts - 1 of one quad, in order.  The loads of up to eight parts are issued
// before the first is used: one after the other they would cost a round trip to L2 each, which
// is most of this kernel's time when a product leaves nine partial sums.
template <typename TD>
__device__ __forceinline__ void add_parts(const TD *dr, int n_parts, long long part_stride, int i, int c1, int vec, float (&d)[PER]) {
    constexpr int AHEAD = 8;
    for (int p0 = 1; p0 < n_parts; p0 += AHEAD) {
        float e[AHEAD][PER];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u)
            if (p0 + u < n_parts) load_quad(dr + (size_t)(p0 + u) * part_stride, i, c1, vec, e[u]);
#pragma unroll
        for (int u = 0; u < AHEAD; ++u)
            if (p0 + u < n_parts) {
#pragma unroll
                for (int q = 0; q < PER; ++q) d[q] += e[u][q];
            }
    }
}

// x + delta of one quad: the parts in order, then the bias; written back unless rows are gathered
template <typename TD>
__device__ __forceinline__ void add_delta(const Args &a, float *xr, const TD *dr, int i, int c1, float (&v)[PER]) {
    float d[PER];
    load_quad(dr, i, c1, a.vec, d);
    add_parts(dr, a.n_parts, a.part_stride, i, c1, a.vec, d);
    if (a.delta_bias) {
        float bq[PER];
        load_quad_const(a.delta_bias, i, c1, a.vec, bq);
#pragma unroll
        for (int q = 0; q < PER; ++q) d[q] += bq[q];
    }
#pragma unroll
    for (int q = 0; q < PER; ++q) v[q] += d[q];
    if (!a.rows) store_quad(xr, i, c1, a.vec, v);
}

// SLICES = 1: this block holds one slice (its cluster rank, or the whole of a narrow row);
// SLICES = MAX_CS: it holds all slices of its row.  ROUNDS rounds of a slice stay in registers.
// FULL: every slice is exactly ROUNDS rounds of whole quads and 16-byte accesses are allowed, so
// no access needs a test (the usual case: widths that are multiples of 512 x slices).
// MODE 0: one block of 128 threads takes SLICES slices of its row; 1: the slices of a row are the
// CTAs of a cluster; 2: the slices of a row are the groups of 128 threads of one block.
template <typename TD, typename TO, int ROUNDS, int SLICES, int MODE, bool FULL>
__global__ void __launch_bounds__(MODE == 2 ? GROUP * MAX_CS : GROUP) rmsnorm_kernel(const Args a) {
    constexpr bool CLUSTERED = MODE == 1;
    constexpr bool GROUPED = MODE == 2;
    pdl_trigger();
    pdl_wait();
    namespace cg = cooperative_groups;
    __shared__ float red[GROUPED ? MAX_CS : SLICES][WARPS];
    __shared__ float slice_ss;
    const int gt = GROUPED ? (threadIdx.x & (GROUP - 1)) : threadIdx.x, cs = a.cs, width = a.width;
    const int r = CLUSTERED ? blockIdx.x / cs : blockIdx.x;
    const int rank0 = CLUSTERED ? blockIdx.x - r * cs : (GROUPED ? threadIdx.x / GROUP : 0);
    const int per_cta = FULL ? ROUNDS * PER * GROUP : (((width + cs - 1) / cs + 3) & ~3);
    const size_t src = a.rows ? (size_t)a.rows[r] : (size_t)r;
    float *xr = a.x + src * width;
    const TD *dr = a.delta ? reinterpret_cast<const TD *>(a.delta) + src * width : nullptr;
    const int n_slices = (CLUSTERED || GROUPED || FULL) ? SLICES : cs;
    const bool vec = FULL ? true : (a.vec != 0);
    // first element of (slice k, round rd) of this thread, and the end of slice k
    auto first = [&](int k, int rd) { return (rank0 + k) * per_cta + rd * PER * GROUP + PER * gt; };
    auto end = [&](int k) { return FULL ? (1 << 30) : (k < n_slices ? min(width, (rank0 + k + 1) * per_cta) : 0); };
    float v[SLICES][ROUNDS][PER];
    // every load of x first
#pragma unroll
    for (int k = 0; k < SLICES; ++k)
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) load_quad(xr, first(k, rd), end(k), vec, v[k][rd]);
    if (dr) {
        // every load of the delta's first part next (no store lies between them), then the
        // other parts in order, the bias, and the sums back to x
        RawQuad<TD> d0[SLICES][ROUNDS];
#pragma unroll
        for (int k = 0; k < SLICES; ++k)
#pragma unroll
            for (int rd = 0; rd < ROUNDS; ++rd) d0[k][rd].load(dr, first(k, rd), end(k), vec);
#pragma unroll
        for (int k = 0; k < SLICES; ++k)
#pragma unroll
            for (int rd = 0; rd < ROUNDS; ++rd) {
                const int c1 = end(k), i = first(k, rd);
                float d[PER];
                d0[k][rd].get(d);
                add_parts(dr, a.n_parts, a.part_stride, i, c1, vec, d);
                if (a.delta_bias) {
                    float bq[PER];
                    load_quad_const(a.delta_bias, i, c1, vec, bq);
#pragma unroll
                    for (int q = 0; q < PER; ++q) d[q] += bq[q];
                }
#pragma unroll
                for (int q = 0; q < PER; ++q) v[k][rd][q] += d[q];
                if (!a.rows) store_quad(xr, i, c1, vec, v[k][rd]);
            }
    }
#pragma unroll
    for (int k = 0; k < SLICES; ++k) {
        float ss = 0.f;
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd)
#pragma unroll
            for (int q = 0; q < PER; ++q) ss = fmaf(v[k][rd][q], v[k][rd][q], ss);
        ss = warp_sum(ss);
        if ((gt & 31) == 0) red[GROUPED ? rank0 : k][gt >> 5] = ss;
    }
    __syncthreads();
    float total = 0.f;
    for (int k = 0; k < (GROUPED ? cs : n_slices); ++k) {
        float slice = 0.f;
        for (int w = 0; w < WARPS; ++w) slice += red[k][w];
        total += slice;
    }
    if (CLUSTERED) {
        cg::cluster_group cluster = cg::this_cluster();
        if (gt == 0) slice_ss = total;
        cluster.sync();
        total = 0.f;
        for (int k = 0; k < cs; ++k) total += *cluster.map_shared_rank(&slice_ss, k);
    }
    const float inv = 1.0f / sqrtf(total / (float)width + a.eps);
    TO *orow = reinterpret_cast<TO *>(a.out) + (size_t)r * width;
#pragma unroll
    for (int k = 0; k < SLICES; ++k)
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) {
            const int c1 = end(k), i = first(k, rd);
            if (i < c1) {
                float w[PER], y[PER];
                load_quad_const(a.weight, i, c1, vec, w);
#pragma unroll
                for (int q = 0; q < PER; ++q) y[q] = v[k][rd][q] * inv * w[q];
                store_quad(orow, i, c1, vec, y);
            }
        }
    if (CLUSTERED) cg::this_cluster().sync();     // no CTA leaves while another may still read its slice's sum
}

// Any width: one block per row walks the slices and their rounds, then the row again.
template <typename TD, typename TO>
__global__ void __launch_bounds__(GROUP) rmsnorm_any_kernel(const Args a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int gt = threadIdx.x, cs = a.cs, width = a.width;
    const int r = blockIdx.x;
    const int per_cta = ((width + cs - 1) / cs + 3) & ~3;
    const size_t src = a.rows ? (size_t)a.rows[r] : (size_t)r;
    float *xr = a.x + src * width;
    const TD *dr = a.delta ? reinterpret_cast<const TD *>(a.delta) + src * width : nullptr;
    float total = 0.f;
    for (int k = 0; k < cs; ++k) {
        const int c0 = k * per_cta, c1 = min(width, c0 + per_cta);
        float ss = 0.f;
        for (int i = c0 + PER * gt; i < c1; i += PER * GROUP) {
            float v[PER];
            load_quad(xr, i, c1, a.vec, v);
            if (dr) add_delta<TD>(a, xr, dr, i, c1, v);
#pragma unroll
            for (int q = 0; q < PER; ++q) ss = fmaf(v[q], v[q], ss);
        }
        total += block_sum(ss, red);
    }
    const float inv = 1.0f / sqrtf(total / (float)width + a.eps);
    TO *orow = reinterpret_cast<TO *>(a.out) + (size_t)r * width;
    Args b = a;
    b.rows = a.rows ? a.rows : reinterpret_cast<const int *>(1);      // second walk: never write x again
    for (int k = 0; k < cs; ++k) {
        const int c0 = k * per_cta, c1 = min(width, c0 + per_cta);
        for (int i = c0 + PER * gt; i < c1; i += PER * GROUP) {
            float v[PER], w[PER], y[PER];
            load_quad(xr, i, c1, a.vec, v);            // with a delta and no row list this is the sum just written
            if (dr && a.rows) add_delta<TD>(b, xr, dr, i, c1, v);
            load_quad_const(a.weight, i, c1, a.vec, w);
#pragma unroll
            for (int q = 0; q < PER; ++q) y[q] = v[q] * inv * w[q];
            store_quad(orow, i, c1, a.vec, y);
        }
    }
}
}  // namespace rms

template <typename TD, typename TO>
static int rmsnorm_launch(const rms::Args &a, int n_rows, cudaStream_t stream) {
    using namespace rms;
    // The number of slices depends on the width only, so a row's sum is formed in the same
    // order whatever else is in the batch.
    const int cs = a.cs;
    const int per_cta = ((a.width + cs - 1) / cs + 3) & ~3;
    const int rounds = (per_cta + PER * GROUP - 1) / (PER * GROUP);
    const bool clustered = cs > 1 && n_rows <= 64;              // many rows fill the GPU without clusters
    cudaError_t e = cudaSuccess;
    // whole quads everywhere: each slice is exactly `rounds` rounds, 16-byte accesses allowed
    const bool full = a.vec && per_cta * cs == a.width && per_cta == rounds * PER * GROUP;
    // LGML_NORM_GROUPED=0: few rows always go to clusters of CTAs (the groups of one block are faster
    // where they fit: 3.3 us against 3.9 us for 8 rows of 4,096 with 9 partial sums)
    static int grouped = -1;
    if (grouped < 0) {
        const char *e = getenv("LGML_NORM_GROUPED");
        grouped = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    if (grouped && clustered && rounds <= 2) {
        const int threads = GROUP * cs;
        if (full && rounds == 1) e = lgml_launch(rmsnorm_kernel<TD, TO, 1, 1, 2, true>, n_rows, threads, 0, stream, a);
        else if (rounds == 1) e = lgml_launch(rmsnorm_kernel<TD, TO, 1, 1, 2, false>, n_rows, threads, 0, stream, a);
        else e = lgml_launch(rmsnorm_kernel<TD, TO, 2, 1, 2, false>, n_rows, threads, 0, stream, a);
    } else if (clustered && rounds <= 4) {
        const int blocks = n_rows * cs;
        if (full && rounds == 1) e = lgml_launch_cluster(rmsnorm_kernel<TD, TO, 1, 1, 1, true>, blocks, GROUP, 0, stream, cs, a);
        else if (full && rounds == 2) e = lgml_launch_cluster(rmsnorm_kernel<TD, TO, 2, 1, 1, true>, blocks, GROUP, 0, stream, cs, a);
        else switch (rounds) {
            case 1: e = lgml_launch_cluster(rmsnorm_kernel<TD, TO, 1, 1, 1, false>, blocks, GROUP, 0, stream, cs, a); break;
            case 2: e = lgml_launch_cluster(rmsnorm_kernel<TD, TO, 2, 1, 1, false>, blocks, GROUP, 0, stream, cs, a); break;
            case 3: e = lgml_launch_cluster(rmsnorm_kernel<TD, TO, 3, 1, 1, false>, blocks, GROUP, 0, stream, cs, a); break;
            default: e = lgml_launch_cluster(rmsnorm_kernel<TD, TO, 4, 1, 1, false>, blocks, GROUP, 0, stream, cs, a); break;
        }
    } else if (cs == 1 && rounds <= 2) {
        if (rounds == 1) e = lgml_launch(rmsnorm_kernel<TD, TO, 1, 1, 0, false>, n_rows, GROUP, 0, stream, a);
        else e = lgml_launch(rmsnorm_kernel<TD, TO, 2, 1, 0, false>, n_rows, GROUP, 0, stream, a);
    } else if (cs == MAX_CS && full && rounds == 1) {
        e = lgml_launch(rmsnorm_kernel<TD, TO, 1, MAX_CS, 0, true>, n_rows, GROUP, 0, stream, a);
    } else if (cs > 1 && rounds <= 2) {
        if (rounds == 1) e = lgml_launch(rmsnorm_kernel<TD, TO, 1, MAX_CS, 0, false>, n_rows, GROUP, 0, stream, a);
        else e = lgml_launch(rmsnorm_kernel<TD, TO, 2, MAX_CS, 0, false>, n_rows, GROUP, 0, stream, a);
    } else {
        e = lgml_launch(rmsnorm_any_kernel<TD, TO>, n_rows, GROUP, 0, stream, a);
    }
    (void)e;
    return lgml_launch_status("rmsnorm");
}

template <typename TD>
static int rmsnorm_dispatch(float *x, const TD *delta, int n_parts, long long part_stride, const float *delta_bias,
                            const float *weight, const int *rows, void *out, int out_dtype, int n_rows, int width, float eps,
                            cudaStream_t stream) {
    rms::Args a;
    a.x = x, a.delta = delta, a.n_parts = n_parts, a.part_stride = part_stride, a.delta_bias = delta_bias, a.weight = weight;
    a.rows = rows, a.out = out, a.width = width, a.eps = eps;
    a.cs = width >= 2048 ? 8 : (width >= 1024 ? 4 : 1);
    const uintptr_t ptrs = (uintptr_t)x | (uintptr_t)delta | (uintptr_t)delta_bias | (uintptr_t)weight | (uintptr_t)out;
    a.vec = (width % 4 == 0 && part_stride % 4 == 0 && (ptrs & 15) == 0) ? 1 : 0;
    if (out_dtype == LGML_F32) return rmsnorm_launch<TD, float>(a, n_rows, stream);
    return rmsnorm_launch<TD, __nv_bfloat16>(a, n_rows, stream);
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
// x *= scale, then x = cap * tanh(x / cap) when cap > 0, in place on float32: the embedding
// scale, the logit scale and the logits' cap that other families of the reference switch on
// (embd_scale lua/lgml/transformer.lua:2303-2306, logit_scale and softcap :2097-2102).  Llama
// uses none of them and never launches this.
// ---------------------------------------------------------------------------------------
__global__ void scale_cap_kernel(float *__restrict__ x, size_t total, float scale, float cap) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = act_load(x + i) * scale;
        if (cap > 0.f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
}

LGML_API int lgml_scale_cap(float *x, long long total, float scale, float cap, cudaStream_t stream) {
    LGML_REQUIRE(total >= 0 && cap >= 0.f, "scale_cap: bad size or a negative cap");
    if (total == 0) return 0;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    lgml_launch(scale_cap_kernel, (int)(want < 148 * 16 ? want : 148 * 16), threads, 0, stream, x, (size_t)total, scale, cap);
    return lgml_launch_status("scale_cap");
}

// ---------------------------------------------------------------------------------------
// Asking L2 for bytes that a later kernel will read (weights): every thread requests chunks
// with cp.async.bulk.prefetch.L2 and the kernel ends; nothing waits for the bytes.  With
// `keep` the lines are marked to be evicted last, so that what streams through L2 before the
// reader comes (the cache's pages) does not push them out; the reader then fetches them with a
// plain load and they age like any other line.  Launched without programmatic serialization:
// it runs on a stream of its own beside the step's chain.
// ---------------------------------------------------------------------------------------
__global__ void l2_ahead_kernel(const char *p, size_t bytes, int keep) {
    const size_t chunk = 16384;
    uint64_t policy = 0;
    if (keep) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    const size_t stride = (size_t)gridDim.x * blockDim.x * chunk;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * chunk; i < bytes; i += stride) {
        const size_t left = bytes - i;
        const unsigned n = (unsigned)((left < chunk ? left : chunk) & ~(size_t)15);
        if (n == 0) break;
        if (keep)
            asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(p + i), "r"(n), "l"(policy) : "memory");
        else
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + i), "r"(n) : "memory");
    }
}

LGML_API int lgml_l2_ahead(const void *p, long long bytes, int keep, cudaStream_t stream) {
    LGML_REQUIRE(bytes >= 0 && ((uintptr_t)p & 15) == 0, "l2_ahead: a negative size or an address off a 16-byte boundary");
    if (bytes < 16) return 0;
    const long long chunks = (bytes + 16383) / 16384;
    const int threads = 128;
    long long blocks = (chunks + threads - 1) / threads;
    if (blocks > 32) blocks = 32;
    l2_ahead_kernel<<<(int)blocks, threads, 0, stream>>>((const char *)p, (size_t)bytes, keep);
    return lgml_launch_status("l2_ahead");
}

// ---------------------------------------------------------------------------------------
// Seeded normal fill: value i of a tensor = mean + sd * z_i, z_i ~ N(0,1) from a counter-based
// stream keyed by (seed, i): splitmix64 of seed and index, then Box-Muller, as mischief/lgml
// fills its test tensors (src/lgml.c:3064-3079, :3133-3137).  The host has the same generator
// (weights/random_init.py) and must draw the same bits, so nothing here comes from a math
// library: the logarithm and the cosine are short polynomials of single, correctly rounded
// float32 operations in a fixed order (the _rn intrinsics are never fused into an FMA), and
// all range reduction is integer arithmetic on the 24-bit uniform numbers.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ULL;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

#define FM(a, b) __fmul_rn((a), (b))
#define FA(a, b) __fadd_rn((a), (b))

// ln(k / 2^24) for an integer 1 <= k <= 2^24: k = m 2^e with m in (sqrt(1/2), sqrt(2)],
// ln m = 2 atanh(s), s = (m - 1) / (m + 1), as an odd series up to s^11
__device__ __forceinline__ float seeded_log_u24(uint32_t k) {
    const uint32_t bits = __float_as_uint((float)k);         // exact: k has at most 25 bits and 2^24 is a power of two
    int e = (int)(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x7fffffu) | 0x3f800000u);              // [1, 2)
    if (m > 0x1.6a09e6p+0f) { m = FM(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(FA(m, -1.0f), FA(m, 1.0f));
    const float s2 = FM(s, s);
    float p = FA(0x1.99999ap-3f, FM(s2, FA(0x1.24924ap-3f, FM(s2, FA(0x1.c71c72p-4f, FM(s2, 0x1.745d18p-4f))))));   // 1/5, 1/7, 1/9, 1/11
    p = FM(s2, FA(0x1.555556p-2f, FM(s2, p)));                                                                       // 1/3
    const float lnm = FM(2.0f, FA(s, FM(s, p)));
    return FA(FM((float)(e - 24), 0x1.62e430p-1f), lnm);                      // + (e - 24) ln 2
}

// cos(2 pi j / 2^24) for an integer 0 <= j < 2^24: the octant and the fold to [0, pi/4] in
// integers, then the Taylor polynomials of sine and cosine
__device__ __forceinline__ float seeded_cos_u24(uint32_t j) {
    const uint32_t q = j >> 21, f = j & 0x1fffffu;
    const uint32_t g = (q & 1u) ? 0x200000u - f : f;         // odd octants run backwards
    const float x = FM((float)g, 0x1.921fb6p-22f);           // pi / 4 / 2^21
    const float x2 = FM(x, x);
    float r;
    if ((q + 1u) & 2u) {                                     // octants 1, 2, 5, 6: the sine
        const float p = FA(-0x1.555556p-3f, FM(x2, FA(0x1.111112p-7f, FM(x2, FA(-0x1.a01a02p-13f, FM(x2, 0x1.71de3ap-19f))))));
        r = FA(x, FM(x, FM(x2, p)));
    } else {
        const float p = FA(-0.5f, FM(x2, FA(0x1.555556p-5f, FM(x2, FA(-0x1.6c16c2p-10f, FM(x2, 0x1.a01a02p-16f))))));
        r = FA(1.0f, FM(x2, p));
    }
    return (q >= 2u && q <= 5u) ? -r : r;
}

__device__ __forceinline__ float seeded_normal(uint64_t seed, uint64_t i) {
    const uint64_t h = splitmix64(seed ^ splitmix64(i));
    const float ln_u = seeded_log_u24((uint32_t)(h >> 40) + 1u);              // u1 in (0, 1]
    const float radius = __fsqrt_rn(FM(-2.0f, ln_u));
    return FM(radius, seeded_cos_u24((uint32_t)(h >> 8) & 0xffffffu));
}

template <typename T>
__global__ void fill_normal_kernel(T *__restrict__ out, size_t n, float mean, float sd, uint64_t seed) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(FA(mean, FM(sd, seeded_normal(seed, i))));
}
#undef FM
#undef FA

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
