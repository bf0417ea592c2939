// The allocation-free variant of the split-KV decode attention (see the header for who
// needs it and for its rules).  It reuses the kernels of attention_decode.cu unchanged by
// including that file, and differs only in where the scratch for the splits' partial
// results lives: a file-scope device array instead of memory from the caller.
#include <atomic>

#include "attention_decode.cu"

#include "attention_decode_noalloc.h"

// The scratch itself.  In host code this name is only a stand-in for the symbol, not a
// device address; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float lgml_noalloc_scratch[LGML_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
// looked up once per device; two threads that look it up at the same time store the same address
std::atomic<float *> scratch_of_device[MAX_DEVICES];

// The device address of the array on the current device; nullptr (and the error text) on failure.
float *noalloc_scratch() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        snprintf(lgml_err_buf, sizeof(lgml_err_buf), "decode_attention_noalloc: cannot tell the current device (%s)",
                 e != cudaSuccess ? cudaGetErrorString(e) : "index out of range");
        return nullptr;
    }
    float *known = scratch_of_device[dev].load(std::memory_order_acquire);
    if (known == nullptr) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, lgml_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            snprintf(lgml_err_buf, sizeof(lgml_err_buf), "decode_attention_noalloc: no address for the scratch array on device %d (%s)",
                     dev, cudaGetErrorString(e));
            return nullptr;
        }
        scratch_of_device[dev].store(ptr, std::memory_order_release);
        known = ptr;
    }
    return known;
}
}  // namespace

LGML_API const char *lgml_attention_decode_noalloc_last_error(void) { return lgml_err_buf; }

LGML_API int lgml_decode_attention_noalloc(const void *q, int ldq, const int *positions, const int *seq_of_token,
                                           const int *block_table, int max_blocks, const void *k_pages, const void *v_pages,
                                           int n_pages, int page_size, void *out, int ldo, int n_splits, int n_tokens, int H,
                                           int Hkv, int D, float scale, int window, int max_new_tokens, int *status,
                                           cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && D > 0 && n_splits >= 1, "decode_attention_noalloc: bad sizes");
    const long long need = lgml_decode_attention_scratch_floats(n_tokens, H, D, n_splits);
    LGML_REQUIRE(need <= (long long)LGML_NOALLOC_SCRATCH_FLOATS,
                 "decode_attention_noalloc: %d tokens x %d heads x %d splits x (%d + 2) = %lld floats of scratch, the built-in array holds %u; "
                 "use fewer splits or tokens per call, or the entry point that takes scratch from the caller",
                 n_tokens, H, n_splits, D, need, (unsigned)LGML_NOALLOC_SCRATCH_FLOATS);
    float *scratch = noalloc_scratch();
    if (scratch == nullptr) return -1;
    return lgml_decode_attention(q, ldq, positions, seq_of_token, block_table, max_blocks, k_pages, v_pages, n_pages, page_size, out,
                                 ldo, scratch, n_splits, n_tokens, H, Hkv, D, scale, window, max_new_tokens, status, stream);
}
