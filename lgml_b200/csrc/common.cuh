// Shared helpers of the sm_100a kernels.  Every launcher is an extern "C" function that
// takes raw device pointers and a stream, launches, and returns 0 or an error code whose
// text lgml_last_error() of the same library gives.  Nothing here allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define LGML_API extern "C" __attribute__((visibility("default")))

// One error string per library (each .cu file is built into its own shared object).
static thread_local char lgml_err_buf[512];

#define LGML_DEFINE_LAST_ERROR(prefix) \
    LGML_API const char *prefix##_last_error(void) { return lgml_err_buf; }

#define LGML_FAIL(...)                                           \
    do {                                                         \
        snprintf(lgml_err_buf, sizeof(lgml_err_buf), __VA_ARGS__); \
        return -1;                                               \
    } while (0)

#define LGML_REQUIRE(cond, ...) \
    do {                        \
        if (!(cond)) LGML_FAIL(__VA_ARGS__); \
    } while (0)

static inline int lgml_launch_status(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(lgml_err_buf, sizeof(lgml_err_buf), "%s: %s", what, cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of this package is launched with the "programmatic stream serialization"
// attribute: the next kernel in the stream may start (its blocks become resident, and may do
// work that does not depend on earlier kernels, such as fetching weights) once all blocks of
// this one have called pdl_trigger().  A kernel calls pdl_wait() before it reads anything an
// earlier kernel wrote and before it writes anything at all; the wait returns when the
// kernels before it have completed and their writes are visible.  Decoding is a chain of many
// short kernels, and this overlaps each kernel's start-up with its predecessor's tail.
// Where the trigger goes: a kernel whose CTAs leave room on their SM (the small kernels, the
// products for few tokens) triggers at its start.  A kernel whose CTAs fill an SM (the products for
// many tokens, alone or in pairs; the tcgen05 prompt attention with all of tensor memory) triggers
// at its end.  Released at its start, the kernels behind it start too, each as soon as the one
// ahead has started, and pile up: CTAs that hold shared and tensor memory while they wait for
// kernels whose own CTAs are not all in yet.  Prompt steps hung that way on the GPU, rarely as the
// kernels were and within a few hundred steps once a small kernel between two large ones did more
// work before its wait; with the attribute off they never did.
// LGML_PDL=0 in the environment turns the attribute off (the instructions are then no-ops).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// A kernel launched this way may already be running while the kernel ahead of it is still
// writing its results.  Its reads of those results therefore go through L2 (ld.global.cg): the
// read-only cache path that the compiler picks for const __restrict__ pointers (ld.global.nc) is
// coherent only at kernel boundaries, and was seen to return the previous layer's values.
// Weights, block tables and other data the stream does not write may still be read any way.
__device__ __forceinline__ float act_load(const float *p) { return __ldcg(p); }
__device__ __forceinline__ __nv_bfloat16 act_load(const __nv_bfloat16 *p) { return __ldcg(p); }
__device__ __forceinline__ unsigned int act_load(const unsigned int *p) { return __ldcg(p); }
__device__ __forceinline__ float2 act_load(const float2 *p) { return __ldcg(p); }
__device__ __forceinline__ float4 act_load(const float4 *p) { return __ldcg(p); }
__device__ __forceinline__ uint4 act_load(const uint4 *p) { return __ldcg(p); }

static inline bool lgml_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char *e = getenv("LGML_PDL");
        enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return enabled != 0;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t lgml_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lgml_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with a thread-block cluster of `cluster` CTAs along x (1: no cluster).
template <typename... KArgs, typename... Args>
static inline cudaError_t lgml_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster,
                                              Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (lgml_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Element types: 0 = float32, 1 = bfloat16.
enum { LGML_F32 = 0, LGML_BF16 = 1 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads in a fixed order (warp trees, then the warps'
// partial sums by index), so that a row's result does not depend on what else is launched.
__device__ __forceinline__ float block_sum(float v, float *smem /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += smem[w];
    return total;
}
