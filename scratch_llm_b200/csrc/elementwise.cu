// Embedding gather, fused residual-add + RMSNorm, gathered final norm, SwiGLU activation.
//
// The residual stream is kept in 32-bit in both precisions; T is the dtype of matrix-product
// operands (float in the 32-bit path, bfloat16 in the serving path).  Formulas restate
// src/scratch_llm/model.py:145-146 (embedding), :158-162 (RMSNorm), :430-435 (residual adds)
// and :229-237 (SwiGLU) of the reference.
#include "common.cuh"

namespace sllm {

// out[n, :] = table[ids[n], :] as float.  One block per token.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int d) {
    const int64_t n = blockIdx.x;
    const T* src = table + (int64_t)ids[n] * d;
    float* dst = out + n * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_float(src[i]);
}

// If delta != nullptr: resid[row] += delta[row] (stored back).  Then
// out[o] = resid[row] * rsqrt(mean(resid[row]^2) + eps) * w, all in 32-bit, rounded once to T.
// index == nullptr: row = o = blockIdx.x.  Otherwise row = index[blockIdx.x], o = blockIdx.x
// and resid is not written (the gathered final norm).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const int* __restrict__ index, const float* __restrict__ w,
                                   float eps, T* __restrict__ out, int d) {
    __shared__ float scratch[33];
    const int64_t o = blockIdx.x;
    const int64_t row = index ? (int64_t)index[o] : o;
    float* x = resid + row * d;
    const T* dl = delta ? delta + row * d : nullptr;
    T* y = out + o * d;
    float ss = 0.f;
    if (dl) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = x[i] + to_float(dl[i]);
            if (!index) x[i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = x[i];
            ss += v * v;
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = x[i];
        if (dl && index) v += to_float(dl[i]);
        y[i] = from_float<T>(v * inv * w[i]);
    }
}

// out[n, f] = silu(gu[n, f]) * gu[n, F + f], silu(z) = z * sigmoid(z), in 32-bit.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t n_rows,
                              int F) {
    const int64_t total = n_rows * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / F;
        const int f = (int)(i - n * F);
        const float g = to_float(gu[n * 2 * F + f]);
        const float u = to_float(gu[n * 2 * F + F + f]);
        const float s = g / (1.0f + expf(-g));
        out[i] = from_float<T>(s * u);
    }
}

}  // namespace sllm

using namespace sllm;

static int norm_threads(int d) {
    int t = 32;
    while (t < 1024 && t * 4 < d) t <<= 1;
    return t;
}

// dtype: 0 = float32, 1 = bfloat16 (of table / delta / out / gu).
SLLM_EXPORT int sllm_embed(const int* ids, const void* table, float* out, int n_tokens, int d,
                           int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0) return (int)cudaErrorInvalidValue;
    const int threads = norm_threads(d);
    if (dtype == 0)
        embed_kernel<float><<<n_tokens, threads, 0, stream>>>(ids, (const float*)table, out, d);
    else if (dtype == 1)
        embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            ids, (const __nv_bfloat16*)table, out, d);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_add_rmsnorm(float* resid, const void* delta, const int* index,
                                 const float* w, float eps, void* out, int n_out, int d,
                                 int dtype, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (d <= 0) return (int)cudaErrorInvalidValue;
    const int threads = norm_threads(d);
    if (dtype == 0)
        add_rmsnorm_kernel<float><<<n_out, threads, 0, stream>>>(
            resid, (const float*)delta, index, w, eps, (float*)out, d);
    else if (dtype == 1)
        add_rmsnorm_kernel<__nv_bfloat16><<<n_out, threads, 0, stream>>>(
            resid, (const __nv_bfloat16*)delta, index, w, eps, (__nv_bfloat16*)out, d);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_swiglu(const void* gu, void* out, int n_rows, int F, int dtype,
                            cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (F <= 0) return (int)cudaErrorInvalidValue;
    const int64_t total = (int64_t)n_rows * F;
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == 0)
        swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gu, (float*)out,
                                                                  n_rows, F);
    else if (dtype == 1)
        swiglu_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_rows, F);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}
