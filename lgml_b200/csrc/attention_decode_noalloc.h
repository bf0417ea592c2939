/*
 * lgml_decode_attention_noalloc: split-KV decode attention for callers that cannot allocate.
 *
 * This entry point has no counterpart in mischief/lgml; it exists for hosts of this
 * library that must not (or cannot) call cudaMalloc: code running inside a region where
 * device allocation is forbidden or would synchronise the device, plug-ins that are handed
 * a fixed arena, and embedders that have already given all free device memory to someone
 * else.  The regular entry point, lgml_decode_attention, needs scratch memory from its
 * caller whenever the keys are cut into more than one range.  This variant brings its own:
 * a fixed array in the library's device image.
 *
 * What the caller still passes: every input and the output, exactly as for
 * lgml_decode_attention, minus the scratch pointer (max_new_tokens is the most tokens one
 * request brings in this step: 1 when decoding).
 *
 * Limits and rules:
 *  - The scratch array holds LGML_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU
 *    whose context loads this library carries that array until the process exits.  A call
 *    that would need more (n_tokens * H * n_splits * (D + 2) floats) is refused with an
 *    error; nothing is launched.
 *  - The first call on a device looks up the array's device address once
 *    (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first
 *    call before any stream capture begins on that device.  The remembered address belongs
 *    to the context that was current then: after cudaDeviceReset, or under a second context
 *    on the same device, it is stale, and this library must be loaded afresh.
 *  - The function calls no cudaMalloc, cudaFree or any other allocating routine.
 *  - All calls share the one array, which keeps whatever the last call left in it.  The
 *    kernels write every partial result they later read, so nothing has to be cleared
 *    between calls.  Two calls that overlap on the GPU (different streams, or a captured
 *    graph replayed next to a live call) race on it: serialise them.
 *
 * Returns 0, or a non-zero code; lgml_attention_decode_noalloc_last_error() gives the text,
 * to the thread that made the failing call only (the text is kept per thread).
 */
#pragma once
#include <cuda_runtime.h>

#define LGML_NOALLOC_SCRATCH_FLOATS (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int lgml_decode_attention_noalloc(const void *q, int ldq, const int *positions, const int *seq_of_token,
                                  const int *block_table, int max_blocks, const void *k_pages, const void *v_pages,
                                  int n_pages, int page_size, void *out, int ldo, int n_splits, int n_tokens, int H,
                                  int Hkv, int D, float scale, int window, int max_new_tokens, int *status, cudaStream_t stream);

const char *lgml_attention_decode_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
