// Rotary position encoding of q and k, and the write of k and v into the paged cache, in
// one pass over the projection's output.  q is rotated (in place, or into its own buffer);
// k is rotated and stored; v is stored (lua/lgml/transformer.lua:1775, :1788 for the
// rotation; :1838-1839 and :2405-2406 for set_rows into the pool; cell of position p =
// table[p / page] * page + p % page, :1126-1133).  Angles are float32: pos * inv_freq[i],
// then sincosf.  The input may also be the float32 partial sums of a projection that was cut
// along K: they are added in order (and the bias after them) as they are read.
#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_rope_cache)

namespace {
constexpr int ITEMS = 256;   // work items (pairs of elements) per block

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
    const int *__restrict__ block_table, int max_blocks, const float *__restrict__ inv_freq, int n_rot, int pairing,
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
    float a = to_f32(act_load(row + d0)), b = to_f32(act_load(row + d1));
    for (int p = 1; p < n_parts; ++p) {
        a += to_f32(act_load(row + (size_t)p * part_stride + d0));
        b += to_f32(act_load(row + (size_t)p * part_stride + d1));
    }
    if (bias) {
        a += bias[col + d0];
        b += bias[col + d1];
    }
    if (fi >= 0) {
        float s, c;
        sincosf((float)pos * inv_freq[fi], &s, &c);
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
    // where this token's k and v go
    const int seq = seq_of_token[t];
    const int blk = pos / page_size;
    int page = -1;
    if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
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

template <typename TS, typename T>
int launch(const void *src, int lds, int n_parts, long long part_stride, const float *bias, void *q_out, int ldq, const int *positions,
           const int *seq_of_token, const int *block_table, int max_blocks, const float *inv_freq, int n_rot, int pairing, void *k_pages,
           void *v_pages, int n_pages, int page_size, int n_tokens, int H, int Hkv, int D, int write_kv, int *status, cudaStream_t stream) {
    const int items = (write_kv ? H + 2 * Hkv : H) * (D / 2);
    dim3 grid(n_tokens, (items + ITEMS - 1) / ITEMS);
    lgml_launch(rope_kv_write_kernel<TS, T>, grid, ITEMS, 0, stream, (const TS *)src, lds, n_parts, part_stride, bias, (T *)q_out, ldq, positions,
                                                            seq_of_token, block_table, max_blocks, inv_freq, n_rot, pairing, (T *)k_pages,
                                                            (T *)v_pages, n_pages, page_size, H, Hkv, D, write_kv, status);
    return lgml_launch_status("rope_kv_write");
}
}  // namespace

// src: [n_parts][n_tokens][(H + 2 Hkv) D] of src_dtype (row stride lds, part_stride elements between
// parts; n_parts > 1 only with float32).  q_out (dtype, row stride ldq) may be src itself when
// n_parts == 1 and the types agree (rotation in place).  The cache has type `dtype`.
LGML_API int lgml_rope_kv_write(const void *src, int src_dtype, int lds, int n_parts, long long part_stride, const float *bias,
                                void *q_out, int dtype, int ldq, const int *positions, const int *seq_of_token,
                                const int *block_table, int max_blocks, const float *inv_freq, int n_rot, int pairing,
                                void *k_pages, void *v_pages, int n_pages, int page_size, int n_tokens, int H, int Hkv, int D,
                                int write_kv, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && page_size > 0 && max_blocks > 0, "rope_kv_write: bad sizes");
    LGML_REQUIRE(D % 2 == 0, "rope_kv_write: head_dim %d must be even", D);
    LGML_REQUIRE(n_rot >= 0 && n_rot <= D && n_rot % 2 == 0, "rope_kv_write: n_rot %d must be even and at most head_dim %d", n_rot, D);
    LGML_REQUIRE(lds >= (H + 2 * Hkv) * D, "rope_kv_write: row stride %d is below (H + 2 Hkv) D = %d", lds, (H + 2 * Hkv) * D);
    LGML_REQUIRE(ldq >= H * D, "rope_kv_write: q row stride %d is below H D = %d", ldq, H * D);
    LGML_REQUIRE(pairing == 0 || pairing == 1, "rope_kv_write: unknown pairing %d", pairing);
    LGML_REQUIRE(n_parts >= 1 && (n_parts == 1 || src_dtype == LGML_F32), "rope_kv_write: partial sums are float32");
    if (n_tokens == 0) return 0;
#define ARGS src, lds, n_parts, part_stride, bias, q_out, ldq, positions, seq_of_token, block_table, max_blocks, inv_freq, n_rot, pairing, \
             k_pages, v_pages, n_pages, page_size, n_tokens, H, Hkv, D, write_kv, status, stream
    if (src_dtype == LGML_F32 && dtype == LGML_F32) return launch<float, float>(ARGS);
    if (src_dtype == LGML_F32 && dtype == LGML_BF16) return launch<float, __nv_bfloat16>(ARGS);
    if (src_dtype == LGML_BF16 && dtype == LGML_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(ARGS);
#undef ARGS
    LGML_FAIL("rope_kv_write: unsupported types (source %d, output %d)", src_dtype, dtype);
}
