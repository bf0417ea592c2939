// True 32-bit matrix product: C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]), float32 operands,
// float32 FMA accumulation, no tensor cores and no reduced-precision mode.  Every output
// element sums its K products in the order k = 0, 1, 2, ... whatever M, N and the tile it
// falls in, so a row's result does not depend on what else is in the batch.  It stands
// where mischief/lgml calls mul_mat with the f32 flag (src/lgml.c:1811-1839).
#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_gemm_f32)

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TO>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float *__restrict__ A, const float *__restrict__ W,
                                                       const float *__restrict__ bias, TO *__restrict__ C, int M, int N, int K,
                                                       int lda, int ldw, int ldc) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // thread's 4x4 patch: rows ty*4.., cols tx*4..
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile: row = tid / 4 (0..63), k = (tid % 4) * 4 .. +3
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + j][lr] = (am < M && k < K) ? act_load(A + (size_t)am * lda + k) : 0.f;
            Ws[lk + j][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            C[(size_t)m * ldc + n] = from_f32<TO>(v);
        }
    }
}
}  // namespace

// out_dtype selects the type C is stored in; the sum itself is float32 in both cases.
LGML_API int lgml_gemm_f32(const float *A, const float *W, const float *bias, void *C, int out_dtype, int M, int N, int K,
                           int lda, int ldw, int ldc, cudaStream_t stream) {
    LGML_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    LGML_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: a leading dimension is smaller than its row");
    if (M == 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    LGML_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is over %d rows", M, 65535 * BM);
    if (out_dtype == LGML_F32)
        lgml_launch(gemm_f32_kernel<float>, grid, 256, 0, stream, A, W, bias, (float *)C, M, N, K, lda, ldw, ldc);
    else if (out_dtype == LGML_BF16)
        lgml_launch(gemm_f32_kernel<__nv_bfloat16>, grid, 256, 0, stream, A, W, bias, (__nv_bfloat16 *)C, M, N, K, lda, ldw, ldc);
    else
        LGML_FAIL("gemm_f32: unknown output type %d", out_dtype);
    return lgml_launch_status("gemm_f32");
}
