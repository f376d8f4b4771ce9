// Y[M, N] = X[M, K] * W[N, K]^T on the CUDA cores with fused multiply-adds in true 32-bit
// (no tensor-core tf32 mode): the matrix product of the 32-bit path, and of sizes that the
// tensor-core kernels refuse.  `y = x @ W.T`, weight stored (out, in):
// src/scratch_llm/model.py:125-133 of the reference.
//
// Every output element is one chain of fmaf over k = 0..K-1 in ascending order, whatever M
// and N are, so a token's result does not depend on what else is in the batch.
#include "common.cuh"

namespace sllm {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ X, const TIn* __restrict__ W, TOut* __restrict__ Y,
                 int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Bs[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int bm = blockIdx.y * BM, bn = blockIdx.x * BN;
    const int lr = tid >> 2, lc = (tid & 3) * 4;  // load: row 0..63, 4 consecutive k
    const int ty = tid >> 4, tx = tid & 15;       // compute: 4x4 outputs
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lc + i;
            const int m = bm + lr, n = bn + lr;
            As[lc + i][lr] = (m < M && k < K) ? to_float(X[(int64_t)m * ldx + k]) : 0.f;
            Bs[lc + i][lr] = (n < N && k < K) ? to_float(W[(int64_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = bm + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = bn + tx * 4 + j;
            if (n < N) Y[(int64_t)m * ldy + n] = from_float<TOut>(acc[i][j]);
        }
    }
}

}  // namespace sllm

using namespace sllm;

// in_dtype / out_dtype: 0 = float32, 1 = bfloat16.  Supported: (0,0), (1,1), (1,0).
SLLM_EXPORT int sllm_gemm_simt(const void* X, const void* W, void* Y, int M, int N, int K,
                               int64_t ldx, int64_t ldw, int64_t ldy, int in_dtype,
                               int out_dtype, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (in_dtype == 0 && out_dtype == 0)
        gemm_simt_kernel<float, float><<<grid, 256, 0, stream>>>(
            (const float*)X, (const float*)W, (float*)Y, M, N, K, ldx, ldw, ldy);
    else if (in_dtype == 1 && out_dtype == 1)
        gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
            (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (__nv_bfloat16*)Y, M, N, K, ldx,
            ldw, ldy);
    else if (in_dtype == 1 && out_dtype == 0)
        gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(
            (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (float*)Y, M, N, K, ldx, ldw, ldy);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}
