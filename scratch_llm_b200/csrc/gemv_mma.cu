// Y[M, N] = X[M, K] * W[N, K]^T for a handful of tokens (M <= 64): the decode step's matrix
// products, which are bound by reading W once from HBM.
//
// `y = x @ W.T`, weight stored (out, in): src/scratch_llm/model.py:125-133 of the reference,
// whose own decode-shape kernels are Triton GEMVs (src/scratch_llm/kernels/gemm/triton/gemv.py)
// and a stub persistent GEMV (csrc/persistent/persistent_gemv_sm90.cu).  With SWIGLU the kernel
// computes silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu] in one pass
// (src/scratch_llm/model.py:236-237).
//
// A CTA of 8 warps owns 16 rows of W (with SWIGLU: 16 gate rows and the 16 up rows that pair
// with them); warp w streams the w-th eighth of K.  W goes from global memory straight into
// tensor-core A fragments with 16-byte loads: lane (g, t) of a warp loads W[row g][k0 + 8t ..
// k0 + 8t + 7] and W[row g + 8][same k], which feeds two m16n8k16 products if the B fragments
// (the tokens' activations) are read with the same permutation of k.  The eight partial sums of
// a CTA are added in warp order, so a token's result does not depend on the batch.
#include "common.cuh"

namespace sllm {

typedef __nv_bfloat16 bf16;
constexpr int GV_WARPS = 8, GV_THREADS = 256, GV_ROWS = 16, GV_UNROLL = 4;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

// MT: number of 8-token tiles (M <= 8 * MT).  NW: W row blocks per CTA (1, or 2 with SWIGLU).
template <int MT, bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(GV_THREADS)
gemv_mma_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, TOut* __restrict__ Y,
                int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy) {
    constexpr int NW = SWIGLU ? 2 : 1;
    __shared__ float red[GV_WARPS][GV_ROWS][8 * MT + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_out = SWIGLU ? N / 2 : N;   // rows of W per block kind = columns of Y
    const int n0 = blockIdx.x * GV_ROWS;
    // this warp's slice of K, in steps of 32
    const int steps_total = (K + 31) / 32;
    const int steps_per_warp = (steps_total + GV_WARPS - 1) / GV_WARPS;
    const int step_begin = warp * steps_per_warp;
    const int step_end = min(steps_total, step_begin + steps_per_warp);

    float acc[NW][MT][4];
#pragma unroll
    for (int b = 0; b < NW; ++b)
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[b][j][e] = 0.f;

    const bf16* wrow[NW][2];
    bool wok[NW][2];
#pragma unroll
    for (int b = 0; b < NW; ++b)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = n0 + g + 8 * h;
            wok[b][h] = r < n_out;
            wrow[b][h] = W + (int64_t)(wok[b][h] ? r + b * n_out : 0) * ldw;
        }
    const bf16* xrow[MT];
    bool xok[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        xok[j] = 8 * j + g < M;
        xrow[j] = X + (int64_t)(xok[j] ? 8 * j + g : 0) * ldx;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 wv[GV_UNROLL][NW][2];
    uint4 xv[GV_UNROLL][MT];
    auto load_w = [&](int s0) {
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int k = (s0 + u) * 32 + 8 * t;
            const bool kin = (s0 + u) < step_end && k < K;   // K is a multiple of 8
#pragma unroll
            for (int b = 0; b < NW; ++b)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    wv[u][b][h] = (kin && wok[b][h]) ? ld_stream16(wrow[b][h] + k) : zero;
        }
    };
    auto load_x = [&](int s0) {
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int k = (s0 + u) * 32 + 8 * t;
            const bool kin = (s0 + u) < step_end && k < K;
#pragma unroll
            for (int j = 0; j < MT; ++j)
                xv[u][j] = (kin && xok[j]) ? *reinterpret_cast<const uint4*>(xrow[j] + k) : zero;
        }
    };
    auto multiply = [&]() {
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u)
#pragma unroll
            for (int b = 0; b < NW; ++b)
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    mma16816(acc[b][j], wv[u][b][0].x, wv[u][b][1].x, wv[u][b][0].y,
                             wv[u][b][1].y, xv[u][j].x, xv[u][j].y);
                    mma16816(acc[b][j], wv[u][b][0].z, wv[u][b][1].z, wv[u][b][0].w,
                             wv[u][b][1].w, xv[u][j].z, xv[u][j].w);
                }
    };
    // The weights of the first steps are requested before the wait for earlier kernels: nothing
    // writes weights, so this part of the stream overlaps the previous kernel's tail.
    if (step_begin < step_end) load_w(step_begin);
    pdl_wait();
    pdl_trigger();
    if (step_begin < step_end) {
        load_x(step_begin);
        multiply();
    }
    for (int s0 = step_begin + GV_UNROLL; s0 < step_end; s0 += GV_UNROLL) {
        load_w(s0);
        load_x(s0);
        multiply();
    }
    // acc[b][j]: e0, e1 = (row g, tokens 8j + 2t, +1); e2, e3 = (row g + 8, same tokens).
    // The warps' partial sums meet in shared memory, one block kind after the other, and are
    // added in warp order.
    constexpr int PER_THREAD = (GV_ROWS * 8 * MT + GV_THREADS - 1) / GV_THREADS;
    float v[NW][PER_THREAD];
#pragma unroll
    for (int b = 0; b < NW; ++b) {
        if (b) __syncthreads();
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                red[warp][g + 8 * (e >> 1)][8 * j + 2 * t + (e & 1)] = acc[b][j][e];
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int idx = tid + i * GV_THREADS;
            const int r = idx % GV_ROWS, tok = idx / GV_ROWS;
            float sum = 0.f;
            if (tok < 8 * MT) {
#pragma unroll
                for (int w = 0; w < GV_WARPS; ++w) sum += red[w][r][tok];
            }
            v[b][i] = sum;
        }
    }
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int idx = tid + i * GV_THREADS;
        const int r = idx % GV_ROWS, tok = idx / GV_ROWS;
        if (tok >= M || n0 + r >= n_out) continue;
        float out = v[0][i];
        if (SWIGLU) {
            // the unfused path rounds gate and up to bfloat16 before the activation
            const float gate = __bfloat162float(__float2bfloat16_rn(v[0][i]));
            const float up = __bfloat162float(__float2bfloat16_rn(v[NW - 1][i]));
            out = gate / (1.0f + expf(-gate)) * up;
        }
        store_out<TOut>(Y + (int64_t)tok * ldy + n0 + r, out);
    }
}

static int g_gemv_pdl = 1;

template <int MT, bool SWIGLU, typename TOut>
static int launch_gemv(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx,
                       int64_t ldw, int64_t ldy, cudaStream_t stream) {
    const int n_out = SWIGLU ? N / 2 : N;
    const int grid = (n_out + GV_ROWS - 1) / GV_ROWS;
    // launched so that it may start while the previous kernel of the stream drains: the kernel
    // requests its first weights, then waits for that kernel (pdl_wait) before it reads X
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GV_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_gemv_pdl;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_mma_kernel<MT, SWIGLU, TOut>, (const bf16*)X,
                                       (const bf16*)W, (TOut*)Y, M, N, K, ldx, ldw, ldy);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

template <bool SWIGLU, typename TOut>
static int pick_mt(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx,
                   int64_t ldw, int64_t ldy, cudaStream_t stream) {
    if (M <= 8) return launch_gemv<1, SWIGLU, TOut>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    if (M <= 16) return launch_gemv<2, SWIGLU, TOut>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    if (M <= 32) return launch_gemv<4, SWIGLU, TOut>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    return launch_gemv<8, SWIGLU, TOut>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_gemv_max_tokens() { return 64; }

// 1 (default): launch with programmatic stream serialization; 0: plain launches.
SLLM_EXPORT void sllm_gemv_set_pdl(int on) { g_gemv_pdl = on ? 1 : 0; }

// X [M, K], W [N, K] bfloat16, rows 16-byte aligned (K, ldx, ldw multiples of 8).
// swiglu = 0: Y [M, N].  swiglu = 1: W = [gate rows; up rows], Y [M, N / 2].
// out_dtype: 0 = float32, 1 = bfloat16.  Sizes this kernel does not take return
// cudaErrorInvalidValue.
SLLM_EXPORT int sllm_gemv_mma(const void* X, const void* W, void* Y, int M, int N, int K,
                              int64_t ldx, int64_t ldw, int64_t ldy, int swiglu, int out_dtype,
                              cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || (swiglu && (N % 2)))
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (swiglu) {
        if (out_dtype == 1) return pick_mt<true, bf16>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
        if (out_dtype == 0) return pick_mt<true, float>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    } else {
        if (out_dtype == 1) return pick_mt<false, bf16>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
        if (out_dtype == 0) return pick_mt<false, float>(X, W, Y, M, N, K, ldx, ldw, ldy, stream);
    }
    return (int)cudaErrorInvalidValue;
}
