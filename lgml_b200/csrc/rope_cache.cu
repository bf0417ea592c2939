// Rotary position encoding of q and k, and the write of k and v into the paged cache, in
// one pass over the projection's output.  q is rotated in place; k is rotated and stored;
// v is stored (lua/lgml/transformer.lua:1775, :1788 for the rotation; :1838-1839 and
// :2405-2406 for set_rows into the pool; cell of position p = table[p / page] * page +
// p % page, :1126-1133).  Angles are float32: pos * inv_freq[i], then sincosf.
#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_rope_cache)

namespace {
// pairing 0: pairs (i, i + n_rot/2) ("half", the order safetensors checkpoints hold);
// pairing 1: pairs (2i, 2i+1) ("adjacent", the reference's "normal" mode on gguf rows).
template <typename T>
__global__ void rope_kv_write_kernel(T *__restrict__ qkv, int ldq, const int *__restrict__ positions,
                                     const int *__restrict__ seq_of_token, const int *__restrict__ block_table,
                                     int max_blocks, const float *__restrict__ inv_freq, int n_rot, int pairing,
                                     T *__restrict__ k_pages, T *__restrict__ v_pages, int n_pages, int page_size,
                                     int H, int Hkv, int D, int write_kv, int *__restrict__ status) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    T *row = qkv + (size_t)t * ldq;
    const int half = n_rot / 2;

    // where this token's k and v go
    const int seq = seq_of_token[t];
    const int blk = pos / page_size;
    int page = -1;
    if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
    const bool ok = write_kv && page >= 0 && page < n_pages;
    if (write_kv && !ok && threadIdx.x == 0) atomicExch(status, 2);  // the host reserves pages first; never write outside the pool
    const size_t cell = ((size_t)(ok ? page : 0) * Hkv) * page_size * D + (size_t)(pos % page_size) * D;

    // rotations: heads 0..H-1 are q, H..H+Hkv-1 are k
    const int n_pairs = (write_kv ? H + Hkv : H) * half;
    for (int w = threadIdx.x; w < n_pairs; w += blockDim.x) {
        const int head = w / half, i = w - head * half;
        const int d0 = pairing ? 2 * i : i, d1 = pairing ? 2 * i + 1 : i + half;
        T *h = row + (size_t)head * D;
        const float a = to_f32(h[d0]), b = to_f32(h[d1]);
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        const float r0 = a * c - b * s, r1 = a * s + b * c;
        if (head < H) {
            h[d0] = from_f32<T>(r0);
            h[d1] = from_f32<T>(r1);
        } else if (ok) {
            T *dst = k_pages + cell + (size_t)(head - H) * page_size * D;
            dst[d0] = from_f32<T>(r0);
            dst[d1] = from_f32<T>(r1);
        }
    }
    if (!ok) return;
    // the part of k past n_rot passes through; v is copied
    for (int w = threadIdx.x; w < Hkv * (D - n_rot); w += blockDim.x) {
        const int g = w / (D - n_rot), d = n_rot + (w - g * (D - n_rot));
        k_pages[cell + (size_t)g * page_size * D + d] = row[(size_t)(H + g) * D + d];
    }
    for (int w = threadIdx.x; w < Hkv * D; w += blockDim.x) {
        const int g = w / D, d = w - g * D;
        v_pages[cell + (size_t)g * page_size * D + d] = row[(size_t)(H + Hkv + g) * D + d];
    }
}
}  // namespace

LGML_API int lgml_rope_kv_write(void *qkv, int dtype, int ldq, const int *positions, const int *seq_of_token,
                                const int *block_table, int max_blocks, const float *inv_freq, int n_rot, int pairing,
                                void *k_pages, void *v_pages, int n_pages, int page_size, int n_tokens, int H, int Hkv, int D,
                                int write_kv, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && page_size > 0 && max_blocks > 0, "rope_kv_write: bad sizes");
    LGML_REQUIRE(n_rot >= 0 && n_rot <= D && n_rot % 2 == 0, "rope_kv_write: n_rot %d must be even and at most head_dim %d", n_rot, D);
    LGML_REQUIRE(ldq >= (H + 2 * Hkv) * D, "rope_kv_write: row stride %d is below (H + 2 Hkv) D = %d", ldq, (H + 2 * Hkv) * D);
    LGML_REQUIRE(pairing == 0 || pairing == 1, "rope_kv_write: unknown pairing %d", pairing);
    if (n_tokens == 0) return 0;
    const int threads = 128;
    if (dtype == LGML_F32)
        rope_kv_write_kernel<float><<<n_tokens, threads, 0, stream>>>((float *)qkv, ldq, positions, seq_of_token, block_table, max_blocks,
                                                                     inv_freq, n_rot, pairing, (float *)k_pages, (float *)v_pages, n_pages,
                                                                     page_size, H, Hkv, D, write_kv, status);
    else if (dtype == LGML_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            (__nv_bfloat16 *)qkv, ldq, positions, seq_of_token, block_table, max_blocks, inv_freq, n_rot, pairing,
            (__nv_bfloat16 *)k_pages, (__nv_bfloat16 *)v_pages, n_pages, page_size, H, Hkv, D, write_kv, status);
    else
        LGML_FAIL("rope_kv_write: unknown type %d", dtype);
    return lgml_launch_status("rope_kv_write");
}
