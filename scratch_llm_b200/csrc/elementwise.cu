// Embedding gather, fused residual-add + RMSNorm, gathered final norm, SwiGLU activation.
//
// The residual stream is kept in 32-bit in both precisions; T is the dtype of matrix-product
// operands (float in the 32-bit path, bfloat16 in the serving path).  Formulas restate
// src/scratch_llm/model.py:145-146 (embedding), :158-162 (RMSNorm), :430-435 (residual adds)
// and :229-237 (SwiGLU) of the reference.
#include "common.cuh"

namespace sllm {

// out[n, :] = table[ids[n], :] as float, times scale.  One block per token.  An id -1 - j stands
// for pending[j]: a token that an earlier kernel of the stream chose and the host has not read yet.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pending,
                             const T* __restrict__ table, float* __restrict__ out, int d,
                             float scale) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    int id = ids[n];
    if (id < 0) id = pending[-1 - id];
    const T* src = table + (int64_t)id * d;
    float* dst = out + n * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
}

// The embedding with the first norm prepared for the product after it (up to 8 tokens, bfloat16
// table): out[n, :] as embed_kernel, x_out[n, i] = bfloat16(out[n, i] * gain[i]), and
// shares[i / 8][n] = sum of out[n, i]^2 over the 8 features of group i / 8: the product that
// follows multiplies its outputs by rsqrt(sum of the shares / d + eps).  One block per token,
// d a multiple of 8.
__global__ void embed_prepare_kernel(const int* __restrict__ ids, const int* __restrict__ pending,
                                     const __nv_bfloat16* __restrict__ table, float* __restrict__ out,
                                     int d, float scale, const float* __restrict__ gain,
                                     __nv_bfloat16* __restrict__ x_out, int64_t ld_xout,
                                     float* __restrict__ shares) {
    pdl_wait();
    pdl_trigger();
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0) id = pending[-1 - id];
    const __nv_bfloat16* src = table + (int64_t)id * d;
    float* dst = out + (int64_t)n * d;
    __nv_bfloat16* xo = x_out + (int64_t)n * ld_xout;
    for (int g = threadIdx.x; g < d / 8; g += blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + g * 8);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = __bfloat162float(e[j]) * scale;
            dst[g * 8 + j] = v;
            xo[g * 8 + j] = __float2bfloat16_rn(v * gain[g * 8 + j]);
            sq += v * v;
        }
        shares[(int64_t)g * 8 + n] = sq;
    }
}

// x = cap * tanh(x * scale / cap) in place (cap > 0), or x * scale (cap == 0): what some
// architectures do to their logits before sampling.
__global__ void logit_cap_kernel(float* __restrict__ x, int64_t n, float scale, float cap) {
    pdl_wait();
    pdl_trigger();
    const float inv = cap > 0.f ? 1.f / cap : 0.f;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float v = x[i] * scale;
        x[i] = cap > 0.f ? cap * tanhf(v * inv) : v;
    }
}

// If delta != nullptr: resid[row] += delta[row] (stored back).  Then
// out[o] = resid[row] * rsqrt(mean(resid[row]^2) + eps) * w, all in 32-bit, rounded once to T.
// index == nullptr: row = o = blockIdx.x.  Otherwise row = index[blockIdx.x], o = blockIdx.x
// and resid is not written (the gathered final norm).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const int* __restrict__ index, const float* __restrict__ w,
                                   float eps, T* __restrict__ out, int d) {
    pdl_wait();
    pdl_trigger();
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
    pdl_wait();
    pdl_trigger();
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

// The same as add_rmsnorm_kernel for d % 4 == 0 and d <= 4 * VEC_CHUNKS * blockDim.x: 16-byte
// accesses, the row stays in registers between the two passes.  The sum of squares is taken
// in the same thread-strided order as in the scalar kernel's formula, in 32-bit.
constexpr int VEC_CHUNKS = 4;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// SPREAD = false: a thread adds up its chunks itself (d up to 4 * VEC_CHUNKS * blockDim.x).
// SPREAD = true: for d <= 4 * VEC_CHUNKS * blockDim.x <= 4096 and many rows.  A thread's chunk c
// stands for thread threadIdx.x + c * blockDim.x of the kernel with SPREAD = false and
// VEC_CHUNKS times as many threads, and the sums are added in exactly that kernel's order, so
// that a row's result is bitwise the same whichever of the two ran it; but blocks are a quarter
// as large, more of them fit on an SM, and their load, sum and store phases overlap.
template <typename T, bool SPREAD>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const int* __restrict__ index, const float* __restrict__ w,
                                       float eps, T* __restrict__ out, int d) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[33];
    const int64_t o = blockIdx.x;
    const int64_t row = index ? (int64_t)index[o] : o;
    float* x = resid + row * d;
    const T* dl = delta ? delta + row * d : nullptr;
    T* y = out + o * d;
    float4 v[VEC_CHUNKS];
    float ss[VEC_CHUNKS];
#pragma unroll
    for (int c = 0; c < VEC_CHUNKS; ++c) {
        const int i = (threadIdx.x + c * blockDim.x) * 4;
        ss[c] = 0.f;
        if (i < d) {
            v[c] = load4(x + i);
            if (dl) {
                const float4 a = load4(dl + i);
                v[c].x += a.x; v[c].y += a.y; v[c].z += a.z; v[c].w += a.w;
                if (!index) store4(x + i, v[c]);
            }
            ss[c] = v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
        }
    }
    float total;
    if (SPREAD) {
        // warp w's chunk c is warp w + c * (blockDim.x / 32) of the wide kernel
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
#pragma unroll
        for (int c = 0; c < VEC_CHUNKS; ++c) {
            const float s = warp_sum(ss[c]);
            if (lane == 0) scratch[warp + c * n_warps] = s;
        }
        __syncthreads();
        if (warp == 0) {
            float t = lane < VEC_CHUNKS * n_warps ? scratch[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) scratch[32] = t;
        }
        __syncthreads();
        total = scratch[32];
    } else {
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < VEC_CHUNKS; ++c) s += ss[c];
        total = block_sum(s, scratch);
    }
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
#pragma unroll
    for (int c = 0; c < VEC_CHUNKS; ++c) {
        const int i = (threadIdx.x + c * blockDim.x) * 4;
        if (i < d) {
            const float4 g = load4(w + i);
            store4(y + i, make_float4(v[c].x * inv * g.x, v[c].y * inv * g.y, v[c].z * inv * g.z,
                                      v[c].w * inv * g.w));
        }
    }
}

// swiglu for F % 8 == 0: 16-byte accesses (bfloat16) / 32-byte (float).
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t n_rows,
                                  int F) {
    pdl_wait();
    pdl_trigger();
    const int per_row = F / 8;
    const int64_t total = n_rows * per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / per_row;
        const int f = (int)(i - n * per_row) * 8;
        const T* g = gu + n * 2 * F + f;
        const T* u = g + F;
        T* o = out + n * F + f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float4 a = load4(g + 4 * h), b = load4(u + 4 * h);
            store4(o + 4 * h, make_float4(a.x / (1.0f + expf(-a.x)) * b.x,
                                          a.y / (1.0f + expf(-a.y)) * b.y,
                                          a.z / (1.0f + expf(-a.z)) * b.z,
                                          a.w / (1.0f + expf(-a.w)) * b.w));
        }
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
// `pending` may be null if no id is negative.
// See embed_prepare_kernel.  n_tokens <= 8; d a multiple of 8; table rows and x_out rows 16-byte
// aligned; shares [d / 8][8].
SLLM_EXPORT int sllm_embed_prepare(const int* ids, const int* pending, const void* table, float* out,
                                   int n_tokens, int d, float scale, const float* gain, void* x_out,
                                   int64_t ld_xout, float* shares, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_tokens > 8 || d <= 0 || (d % 8) || ((uintptr_t)table & 15)) return (int)cudaErrorInvalidValue;
    int threads = 32;
    while (threads < 1024 && threads * 8 < d) threads <<= 1;
    embed_prepare_kernel<<<n_tokens, threads, 0, stream>>>(
        ids, pending, (const __nv_bfloat16*)table, out, d, scale, gain, (__nv_bfloat16*)x_out,
        ld_xout, shares);
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_logit_cap(float* x, int64_t n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (cap < 0.f) return (int)cudaErrorInvalidValue;
    const int blocks = (int)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    logit_cap_kernel<<<blocks, 256, 0, stream>>>(x, n, scale, cap);
    SLLM_LAUNCH_CHECK();
    return 0;
}

SLLM_EXPORT int sllm_embed(const int* ids, const int* pending, const void* table, float* out,
                           int n_tokens, int d, int dtype, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0) return (int)cudaErrorInvalidValue;
    const int threads = norm_threads(d);
    if (dtype == 0)
        embed_kernel<float><<<n_tokens, threads, 0, stream>>>(ids, pending, (const float*)table, out,
                                                              d, scale);
    else if (dtype == 1)
        embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            ids, pending, (const __nv_bfloat16*)table, out, d, scale);
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
    if (d % 4 == 0 && d <= 4 * VEC_CHUNKS * 1024 && dtype >= 0 && dtype <= 1) {
        int vt = 32;
        while (vt < 1024 && vt * 4 * (d > 4096 ? VEC_CHUNKS : 1) < d) vt <<= 1;
        cudaError_t e;
        // many rows: blocks a quarter as wide with the same (bitwise) result, see the kernel
        const bool spread = d <= 4096 && vt >= 32 * VEC_CHUNKS && n_out >= 296;
        if (spread) vt /= VEC_CHUNKS;
        if (dtype == 0)
            e = spread
                ? sllm_launch_pdl(add_rmsnorm_vec_kernel<float, true>, dim3(n_out), dim3(vt), 0,
                                  stream, resid, (const float*)delta, index, w, eps, (float*)out, d)
                : sllm_launch_pdl(add_rmsnorm_vec_kernel<float, false>, dim3(n_out), dim3(vt), 0,
                                  stream, resid, (const float*)delta, index, w, eps, (float*)out, d);
        else
            e = spread
                ? sllm_launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16, true>, dim3(n_out),
                                  dim3(vt), 0, stream, resid, (const __nv_bfloat16*)delta, index, w,
                                  eps, (__nv_bfloat16*)out, d)
                : sllm_launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16, false>, dim3(n_out),
                                  dim3(vt), 0, stream, resid, (const __nv_bfloat16*)delta, index, w,
                                  eps, (__nv_bfloat16*)out, d);
        return (int)e;
    }
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
    const int threads = 256;
    if (F % 8 == 0 && dtype >= 0 && dtype <= 1) {
        int64_t vblocks = ((int64_t)n_rows * (F / 8) + threads - 1) / threads;
        if (vblocks > 148 * 16) vblocks = 148 * 16;
        if (dtype == 0)
            swiglu_vec_kernel<float><<<(int)vblocks, threads, 0, stream>>>(
                (const float*)gu, (float*)out, n_rows, F);
        else
            swiglu_vec_kernel<__nv_bfloat16><<<(int)vblocks, threads, 0, stream>>>(
                (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_rows, F);
        SLLM_LAUNCH_CHECK();
        return 0;
    }
    const int64_t total = (int64_t)n_rows * F;
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
