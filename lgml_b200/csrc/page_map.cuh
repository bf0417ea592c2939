// TMA descriptors of the paged cache, shared by the attention kernels that copy pages with
// cp.async.bulk.tensor.
#pragma once
#include <cuda.h>

#include "common.cuh"

typedef CUresult (*LgmlEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                      const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline LgmlEncodeTiledFn lgml_encode_tiled() {
    static LgmlEncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (LgmlEncodeTiledFn)ptr;
    }
    return fn;
}

// The cache of one layer, [pages][KV heads][64][D] bfloat16, as a 3-dimensional tensor
// (D, 64, pages x KV heads) read in boxes of 64 columns x 64 rows with the 128-byte swizzle.
// D must be a multiple of 64 (the box starts at columns 0, 64, ...: 16-byte aligned).
static inline int lgml_make_page_map(CUtensorMap *map, const void *base, int n_pages, int Hkv, int D, const char *who) {
    LgmlEncodeTiledFn enc = lgml_encode_tiled();
    if (enc == nullptr) LGML_FAIL("%s: the driver has no cuTensorMapEncodeTiled", who);
    cuuint64_t dims[3] = {(cuuint64_t)D, 64, (cuuint64_t)n_pages * (cuuint64_t)Hkv};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)64 * D * 2};
    cuuint32_t box[3] = {64, 64, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) LGML_FAIL("%s: cuTensorMapEncodeTiled failed with %d (pages %d, KV heads %d, head_dim %d)", who, (int)r, n_pages, Hkv, D);
    return 0;
}
