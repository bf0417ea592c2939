// Rotary position encoding of q and k, and the write of k and v into the paged cache, in
// one pass over the projection's output.  q is rotated (in place, or into its own buffer);
// k is rotated and stored; v is stored (lua/lgml/transformer.lua:1775, :1788 for the
// rotation; :1838-1839 and :2405-2406 for set_rows into the pool; cell of position p =
// table[p / page] * page + p % page, :1126-1133).  Angles are formed in float32 arithmetic
// without losing what a single float32 product would (rope_sincos).  The input may also be the float32 partial sums of a projection that was cut
// along K: they are added in order (and the bias after them) as they are read.
#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_rope_cache)

namespace {
constexpr int ITEMS = 256;   // work items (pairs of elements) per block

// sin and cos of pos * (f + f_lo).  The product of a position in the thousands and a float32
// frequency is thousands of radians, and rounding it to float32 would cost 1e-4 to 1e-3 of a
// radian there.  So: the rounded product a, its exact error (one fma), the frequency's low
// part (what float32 lost of the float64 table; 0 when the caller has none), and a taken
// modulo 2 pi exactly (2 pi in three float32 pieces; the first difference is exact for
// positions below 2^24) before the small terms are added.  All of it float32 operations.
__device__ __forceinline__ void rope_sincos(int pos, float f, float f_lo, float *s, float *c) {
    const float p = (float)pos;
    const float a = __fmul_rn(p, f);
    const float e = fmaf(p, f_lo, fmaf(p, f, -a));
    const float k = rintf(a * 0x1.45f306p-3f);
    float r = fmaf(-k, 0x1.921fb6p+2f, a);
    r = fmaf(-k, -0x1.777a5cp-23f, r);
    r = fmaf(-k, -0x1.ee59dap-48f, r);
    sincosf(r + e, s, c);
}

// One work item = one pair of elements of one head of one token.
//   heads 0 .. H-1: q, rotated, written to q_out;   H .. H+Hkv-1: k, rotated, to the cache;
//   H+Hkv .. H+2Hkv-1: v, copied to the cache.
// pairing 0: pairs (i, i + n_rot/2) ("half", the order safetensors checkpoints hold);
// pairing 1: pairs (2i, 2i+1) ("adjacent", the reference's "normal" mode on gguf rows).
// Dimensions at and past n_rot are paired (2j, 2j+1) and pass through unrotated.
template <typename TS, typename T>
__global__ void __launch_bounds__(ITEMS) rope_kv_write_kernel(
    const TS *__restrict__ src, int lds, int n_parts, long long part_stride, const float *__restrict__ bias,
    T *__restrict__ q_out, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const float *__restrict__ inv_freq, const float *__restrict__ inv_freq_lo, int n_rot, int pairing,
    T *__restrict__ k_pages, T *__restrict__ v_pages, int n_pages, int page_size, int H, int Hkv, int D, int write_kv,
    int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int half_d = D / 2;
    const int n_heads = write_kv ? H + 2 * Hkv : H;
    const int item = blockIdx.y * ITEMS + threadIdx.x;
    if (item >= n_heads * half_d) return;
    const int head = item / half_d, j = item - head * half_d;
    const int pos = positions[t];
    const int half_rot = n_rot / 2;

    // which two dimensions, and whether they turn
    int d0, d1, fi = -1;
    if (head < H + Hkv && j < half_rot) {
        fi = j;
        d0 = pairing ? 2 * j : j;
        d1 = pairing ? 2 * j + 1 : j + half_rot;
    } else if (head < H + Hkv) {
        d0 = n_rot + 2 * (j - half_rot);
        d1 = d0 + 1;
    } else {
        d0 = 2 * j;
        d1 = d0 + 1;
    }
    const size_t col = (size_t)head * D;
    const TS *row = src + (size_t)t * lds + col;
    // Every load goes out before anything waits for one: the elements and their other parts, the
    // bias, the frequency, and the chain position -> block -> page for the cell of the cache (two
    // trips to L2 one after the other, which used to begin only when the rotation was done).
    float a = to_f32(act_load(row + d0)), b = to_f32(act_load(row + d1));
    const float bias0 = bias ? bias[col + d0] : 0.f, bias1 = bias ? bias[col + d1] : 0.f;
    const float f = fi >= 0 ? inv_freq[fi] : 0.f, f_lo = (fi >= 0 && inv_freq_lo) ? inv_freq_lo[fi] : 0.f;
    int page = -1;      // where this token's k and v go
    if (head >= H) {
        const int seq = seq_of_token[t];
        const int blk = pos / page_size;
        if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
    }
    // the other parts in order; the loads of up to eight of them are issued before the first is used
    // (one after the other they would cost a round trip to L2 each)
    for (int p0 = 1; p0 < n_parts; p0 += 8) {
        float ea[8], eb[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (p0 + u < n_parts) {
                ea[u] = to_f32(act_load(row + (size_t)(p0 + u) * part_stride + d0));
                eb[u] = to_f32(act_load(row + (size_t)(p0 + u) * part_stride + d1));
            }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (p0 + u < n_parts) {
                a += ea[u];
                b += eb[u];
            }
    }
    a += bias0;
    b += bias1;
    if (fi >= 0) {
        float s, c;
        rope_sincos(pos, f, f_lo, &s, &c);
        const float r0 = a * c - b * s, r1 = a * s + b * c;
        a = r0;
        b = r1;
    }
    if (head < H) {
        T *dst = q_out + (size_t)t * ldq + col;
        dst[d0] = from_f32<T>(a);
        dst[d1] = from_f32<T>(b);
        return;
    }
    if (page < 0 || page >= n_pages) {   // the host reserves pages first; never write outside the pool
        if (j == 0) atomicExch(status, 2);
        return;
    }
    const bool is_k = head < H + Hkv;
    const int g = is_k ? head - H : head - H - Hkv;
    T *dst = (is_k ? k_pages : v_pages) + (((size_t)page * Hkv + g) * page_size + (size_t)(pos % page_size)) * D;
    dst[d0] = from_f32<T>(a);
    dst[d1] = from_f32<T>(b);
}


// The same for many tokens at once (prompts), bfloat16 in and out, one part: a block per token.
// The token's cosines and sines are computed once and shared by all its heads, and a work unit
// is 16 bytes (8 elements) of one head, or for the "half" pairing the two 16-byte runs that
// hold 8 pairs, so that loads and stores are as wide as the hardware takes.  The arithmetic of
// one pair is that of the kernel above.
constexpr int WIDE_THREADS = 128;
constexpr int WIDE_MAX_ROT = 512;
__global__ void __launch_bounds__(WIDE_THREADS) rope_kv_write_wide_kernel(
    const __nv_bfloat16 *__restrict__ src, int lds, const float *__restrict__ bias, __nv_bfloat16 *__restrict__ q_out, int ldq,
    const int *__restrict__ positions, const int *__restrict__ seq_of_token, const int *__restrict__ block_table, int max_blocks,
    const float *__restrict__ inv_freq, const float *__restrict__ inv_freq_lo, int n_rot, int pairing, __nv_bfloat16 *__restrict__ k_pages,
    __nv_bfloat16 *__restrict__ v_pages, int n_pages, int page_size, int H, int Hkv, int D, int write_kv, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float2 cs[WIDE_MAX_ROT / 2];      // (cos, sin) of pair i
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[t];
    const int half_rot = n_rot / 2;
    for (int i = tid; i < half_rot; i += WIDE_THREADS) {
        float sn, c;
        rope_sincos(pos, inv_freq[i], inv_freq_lo ? inv_freq_lo[i] : 0.f, &sn, &c);
        cs[i] = make_float2(c, sn);
    }
    // where this token's k and v go
    int page = -1;
    if (write_kv) {
        const int seq = seq_of_token[t];
        const int blk = pos / page_size;
        if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
        if (page < 0 || page >= n_pages) {   // the host reserves pages first; never write outside the pool
            if (tid == 0) atomicExch(status, 2);
            page = -1;
        }
    }
    __syncthreads();
    const int rot_units = pairing ? n_rot / 8 : n_rot / 16;     // units of a rotated head that turn
    const int copy_units = (D - n_rot) / 8;                     // and those that pass through
    const int units_qk = rot_units + copy_units, units_v = D / 8;
    const int n_qk = write_kv ? H + Hkv : H;
    const int total = n_qk * units_qk + (write_kv ? Hkv * units_v : 0);
    const __nv_bfloat16 *row = src + (size_t)t * lds;
    for (int u = tid; u < total; u += WIDE_THREADS) {
        int head, unit;
        bool is_v = false;
        if (u < n_qk * units_qk) {
            head = u / units_qk;
            unit = u - head * units_qk;
        } else {
            const int w = u - n_qk * units_qk;
            head = H + Hkv + w / units_v;
            unit = w - (w / units_v) * units_v;
            is_v = true;
        }
        const size_t col = (size_t)head * D;
        __nv_bfloat16 *dst;
        if (head < H) {
            dst = q_out + (size_t)t * ldq + col;
        } else {
            if (page < 0) continue;
            const int g = is_v ? head - H - Hkv : head - H;
            dst = (is_v ? v_pages : k_pages) + (((size_t)page * Hkv + g) * page_size + (size_t)(pos % page_size)) * D;
        }
        if (is_v || unit >= rot_units) {
            // 8 elements that do not turn
            const int d = is_v ? unit * 8 : n_rot + (unit - rot_units) * 8;
            uint4 raw = act_load(reinterpret_cast<const uint4 *>(row + col + d));
            if (bias) {
                __nv_bfloat16 *e = reinterpret_cast<__nv_bfloat16 *>(&raw);
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16_rn(__bfloat162float(e[j]) + bias[col + d + j]);
            }
            *reinterpret_cast<uint4 *>(dst + d) = raw;
        } else if (pairing) {
            // adjacent pairs: 8 elements = pairs 4 unit .. 4 unit + 3
            const int d = unit * 8;
            uint4 raw = act_load(reinterpret_cast<const uint4 *>(row + col + d));
            __nv_bfloat16 *e = reinterpret_cast<__nv_bfloat16 *>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float a = __bfloat162float(e[2 * j]), b = __bfloat162float(e[2 * j + 1]);
                if (bias) {
                    a += bias[col + d + 2 * j];
                    b += bias[col + d + 2 * j + 1];
                }
                const float2 f = cs[unit * 4 + j];
                e[2 * j] = __float2bfloat16_rn(a * f.x - b * f.y);
                e[2 * j + 1] = __float2bfloat16_rn(a * f.y + b * f.x);
            }
            *reinterpret_cast<uint4 *>(dst + d) = raw;
        } else {
            // half pairs: elements 8 unit .. 8 unit + 7 with their partners n_rot / 2 further
            const int d0 = unit * 8, d1 = d0 + half_rot;
            uint4 ra = act_load(reinterpret_cast<const uint4 *>(row + col + d0));
            uint4 rb = act_load(reinterpret_cast<const uint4 *>(row + col + d1));
            __nv_bfloat16 *ea = reinterpret_cast<__nv_bfloat16 *>(&ra), *eb = reinterpret_cast<__nv_bfloat16 *>(&rb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float a = __bfloat162float(ea[j]), b = __bfloat162float(eb[j]);
                if (bias) {
                    a += bias[col + d0 + j];
                    b += bias[col + d1 + j];
                }
                const float2 f = cs[d0 + j];
                ea[j] = __float2bfloat16_rn(a * f.x - b * f.y);
                eb[j] = __float2bfloat16_rn(a * f.y + b * f.x);
            }
            *reinterpret_cast<uint4 *>(dst + d0) = ra;
            *reinterpret_cast<uint4 *>(dst + d1) = rb;
        }
    }
}

// Whether the wide kernel can take this call: 16-byte runs everywhere.
inline bool wide_ok(const void *src, int lds, const void *q_out, int ldq, const void *k_pages, const void *v_pages, int n_rot, int pairing,
                    int D, int n_tokens) {
    if (n_tokens < 32 || n_rot > WIDE_MAX_ROT) return false;
    if (D % 8 || lds % 8 || ldq % 8 || n_rot % (pairing ? 8 : 16)) return false;
    return (((uintptr_t)src | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
}

template <typename TS, typename T>
int launch(const void *src, int lds, int n_parts, long long part_stride, const float *bias, void *q_out, int ldq, const int *positions,
           const int *seq_of_token, const int *block_table, int max_blocks, const float *inv_freq, const float *inv_freq_lo, int n_rot, int pairing,
           void *k_pages, void *v_pages, int n_pages, int page_size, int n_tokens, int H, int Hkv, int D, int write_kv, int *status,
           cudaStream_t stream) {
    const int items = (write_kv ? H + 2 * Hkv : H) * (D / 2);
    dim3 grid(n_tokens, (items + ITEMS - 1) / ITEMS);
    lgml_launch(rope_kv_write_kernel<TS, T>, grid, ITEMS, 0, stream, (const TS *)src, lds, n_parts, part_stride, bias, (T *)q_out, ldq, positions,
                                                            seq_of_token, block_table, max_blocks, inv_freq, inv_freq_lo, n_rot, pairing, (T *)k_pages,
                                                            (T *)v_pages, n_pages, page_size, H, Hkv, D, write_kv, status);
    return lgml_launch_status("rope_kv_write");
}
}  // namespace

// src: [n_parts][n_tokens][(H + 2 Hkv) D] of src_dtype (row stride lds, part_stride elements between
// parts; n_parts > 1 only with float32).  q_out (dtype, row stride ldq) may be src itself when
// n_parts == 1 and the types agree (rotation in place).  The cache has type `dtype`.
// inv_freq: n_rot / 2 frequencies; inv_freq_lo: what float32 lost of each (table - (float)table), or null.
LGML_API int lgml_rope_kv_write(const void *src, int src_dtype, int lds, int n_parts, long long part_stride, const float *bias,
                                void *q_out, int dtype, int ldq, const int *positions, const int *seq_of_token,
                                const int *block_table, int max_blocks, const float *inv_freq, const float *inv_freq_lo, int n_rot,
                                int pairing, void *k_pages, void *v_pages, int n_pages, int page_size, int n_tokens, int H, int Hkv, int D,
                                int write_kv, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && page_size > 0 && max_blocks > 0, "rope_kv_write: bad sizes");
    LGML_REQUIRE(D % 2 == 0, "rope_kv_write: head_dim %d must be even", D);
    LGML_REQUIRE(n_rot >= 0 && n_rot <= D && n_rot % 2 == 0, "rope_kv_write: n_rot %d must be even and at most head_dim %d", n_rot, D);
    LGML_REQUIRE(lds >= (H + 2 * Hkv) * D, "rope_kv_write: row stride %d is below (H + 2 Hkv) D = %d", lds, (H + 2 * Hkv) * D);
    LGML_REQUIRE(ldq >= H * D, "rope_kv_write: q row stride %d is below H D = %d", ldq, H * D);
    LGML_REQUIRE(pairing == 0 || pairing == 1, "rope_kv_write: unknown pairing %d", pairing);
    LGML_REQUIRE(n_parts >= 1 && (n_parts == 1 || src_dtype == LGML_F32), "rope_kv_write: partial sums are float32");
    if (n_tokens == 0) return 0;
#define ARGS src, lds, n_parts, part_stride, bias, q_out, ldq, positions, seq_of_token, block_table, max_blocks, inv_freq, inv_freq_lo, n_rot, pairing, \
             k_pages, v_pages, n_pages, page_size, n_tokens, H, Hkv, D, write_kv, status, stream
    if (src_dtype == LGML_F32 && dtype == LGML_F32) return launch<float, float>(ARGS);
    if (src_dtype == LGML_F32 && dtype == LGML_BF16) return launch<float, __nv_bfloat16>(ARGS);
    if (src_dtype == LGML_BF16 && dtype == LGML_BF16) {
        if (n_parts == 1 && wide_ok(src, lds, q_out, ldq, k_pages, v_pages, n_rot, pairing, D, n_tokens)) {
            lgml_launch(rope_kv_write_wide_kernel, dim3(n_tokens), WIDE_THREADS, 0, stream, (const __nv_bfloat16 *)src, lds, bias,
                        (__nv_bfloat16 *)q_out, ldq, positions, seq_of_token, block_table, max_blocks, inv_freq, inv_freq_lo, n_rot, pairing,
                        (__nv_bfloat16 *)k_pages, (__nv_bfloat16 *)v_pages, n_pages, page_size, H, Hkv, D, write_kv, status);
            return lgml_launch_status("rope_kv_write");
        }
        return launch<__nv_bfloat16, __nv_bfloat16>(ARGS);
    }
#undef ARGS
    LGML_FAIL("rope_kv_write: unsupported types (source %d, output %d)", src_dtype, dtype);
}
