// Causal attention of a packed batch over the paged cache, on the CUDA cores in 32-bit
// arithmetic.  One kernel serves portions of prompts and single decoded tokens: the token at
// absolute position p of row r attends to keys 0..p of row r (or to the last `window` of
// them) through r's block table.  This is the attention of the 32-bit path for every head
// size, and of the bfloat16 path where no tensor-core kernel takes the shape.
//
// Restates src/scratch_llm/model.py:172-182 (scores = q k^T scaled, disallowed keys -inf,
// max-subtracted softmax in 32-bit, times v) and :330-345 (query head h reads kv head
// h / (H/G); key j is visible to the query at position p iff j <= p) of the reference, with
// the online softmax of its paged kernel (src/scratch_llm/kernels/attention/decode/paged.py:49-83).
//
// Keys are consumed in tiles of 32 that are aligned to absolute positions, in ascending
// order, so a query's result does not depend on how its prompt was cut or on its neighbours.
// Compiled once per head size: -DSLLM_HEAD_DIM=<multiple of 16>.
#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#error "compile with -DSLLM_HEAD_DIM=<head size>"
#endif

namespace sllm {

constexpr int HD = SLLM_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 512, "head size: a multiple of 16 up to 512");
constexpr int BQ = 16, BKV = 32, THREADS = 128, ROWS_PER_WARP = 4;
constexpr int DPL = (HD + 31) / 32;  // head dims per lane
constexpr int KS_LD = HD + 1;

constexpr size_t smem_floats() {
    return (size_t)BQ * HD + (size_t)BKV * KS_LD + (size_t)BKV * HD + (size_t)BQ * BKV;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_simt_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ pages,
                 const int* __restrict__ block_table, int table_stride, int page_size,
                 const int* __restrict__ row_start, const int* __restrict__ row_pos0,
                 T* __restrict__ out, int64_t out_stride, int H, int G, float scale, int window) {
    extern __shared__ float smem[];
    __shared__ long long key_base[BKV];  // element offset of each key's K row, -1 if absent
    float* Qs = smem;
    float* Ks = Qs + BQ * HD;
    float* Vs = Ks + BKV * KS_LD;
    float* Ss = Vs + BKV * HD;

    const int r = blockIdx.y, h = blockIdx.z;
    const int g = h / (H / G);
    const int t0 = row_start[r];
    const int n_new = row_start[r + 1] - t0;
    const int q0 = blockIdx.x * BQ;
    if (q0 >= n_new) return;
    const int nq = min(BQ, n_new - q0);
    const int first_pos = row_pos0[r] + q0;
    const int last_pos = first_pos + nq - 1;
    int k_lo = 0;
    if (window > 0) k_lo = max(0, first_pos - window + 1) / BKV * BKV;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int idx = tid; idx < BQ * HD; idx += THREADS) {
        const int i = idx / HD, d = idx - i * HD;
        Qs[idx] = i < nq ? to_float(q[(int64_t)(t0 + q0 + i) * q_stride + (int64_t)h * HD + d])
                         : 0.f;
    }

    float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][DPL];
#pragma unroll
    for (int a = 0; a < ROWS_PER_WARP; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[a][c] = 0.f;
    }
    const int64_t v_offset = (int64_t)G * page_size * HD;

    for (int kt = k_lo; kt <= last_pos; kt += BKV) {
        __syncthreads();  // the previous tile's Ks / Vs / key_base are no longer read
        if (tid < BKV) {
            const int kpos = kt + tid;
            long long base = -1;
            if (kpos <= last_pos) {
                const int page = block_table[(int64_t)r * table_stride + kpos / page_size];
                if (page >= 0)
                    base = (((long long)page * 2 * G + g) * page_size + kpos % page_size) * HD;
            }
            key_base[tid] = base;
        }
        __syncthreads();
        for (int idx = tid; idx < BKV * HD; idx += THREADS) {
            const int j = idx / HD, d = idx - j * HD;
            const long long base = key_base[j];
            float kv = 0.f, vv = 0.f;
            if (base >= 0) {
                kv = to_float(pages[base + d]);
                vv = to_float(pages[base + v_offset + d]);
            }
            Ks[j * KS_LD + d] = kv;
            Vs[j * HD + d] = vv;
        }
        __syncthreads();

        const int kpos = kt + lane;
#pragma unroll
        for (int a = 0; a < ROWS_PER_WARP; ++a) {
            const int i = warp + 4 * a;
            const float* qi = Qs + i * HD;
            const float* kj = Ks + lane * KS_LD;
            float dot = 0.f;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) dot = fmaf(qi[d], kj[d], dot);
            const int qpos = first_pos + i;
            const bool valid = i < nq && kpos <= qpos && (window <= 0 || kpos > qpos - window) &&
                               key_base[lane] >= 0;
            const float s = valid ? dot * scale : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max(s));
            float p = 0.f, corr = 1.f;
            if (m_new != -INFINITY) {
                p = expf(s - m_new);        // s = -inf gives 0
                corr = expf(m[a] - m_new);  // m = -inf gives 0
            }
            l[a] = l[a] * corr + warp_sum(p);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[a][c] *= corr;
            Ss[i * BKV + lane] = p;
        }
        __syncwarp();  // each warp reads back only the rows of Ss it wrote
#pragma unroll
        for (int a = 0; a < ROWS_PER_WARP; ++a) {
            const float* pi = Ss + (warp + 4 * a) * BKV;
            for (int j = 0; j < BKV; ++j) {
                const float p = pi[j];
#pragma unroll
                for (int c = 0; c < DPL; ++c) {
                    const int d = lane + 32 * c;
                    if (d < HD) acc[a][c] = fmaf(p, Vs[j * HD + d], acc[a][c]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < ROWS_PER_WARP; ++a) {
        const int i = warp + 4 * a;
        if (i >= nq) continue;
        const float inv = l[a] > 0.f ? 1.0f / l[a] : 0.f;
        T* o = out + (int64_t)(t0 + q0 + i) * out_stride + (int64_t)h * HD;
#pragma unroll
        for (int c = 0; c < DPL; ++c) {
            const int d = lane + 32 * c;
            if (d < HD) o[d] = from_float<T>(acc[a][c] * inv);
        }
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attn_simt_head_dim() { return HD; }

// q: [n_tokens, q_stride] with head h at columns [h*HD, (h+1)*HD); out likewise.
// pages: [n_pages, 2, G, page_size, HD].  block_table: [n_rows, table_stride], -1 = no page.
// row_start: [n_rows + 1] token offsets; row_pos0: [n_rows] position of each row's first token.
// max_new: the largest number of new tokens of any row.  window: 0 = all keys.
SLLM_EXPORT int sllm_attn_simt(const void* q, int64_t q_stride, const void* pages,
                               const int* block_table, int table_stride, int page_size,
                               const int* row_start, const int* row_pos0, void* out,
                               int64_t out_stride, int n_rows, int max_new, int H, int G,
                               float scale, int window, int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || max_new <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || page_size <= 0 || window < 0)
        return (int)cudaErrorInvalidValue;
    if (n_rows > 65535 || H > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = smem_floats() * sizeof(float);
    dim3 grid((max_new + BQ - 1) / BQ, n_rows, H);
    cudaError_t e;
    if (dtype == 0) {
        e = cudaFuncSetAttribute(attn_simt_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attn_simt_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_stride, (const float*)pages, block_table, table_stride, page_size,
            row_start, row_pos0, (float*)out, out_stride, H, G, scale, window);
    } else if (dtype == 1) {
        e = cudaFuncSetAttribute(attn_simt_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attn_simt_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_table,
            table_stride, page_size, row_start, row_pos0, (__nv_bfloat16*)out, out_stride, H, G,
            scale, window);
    } else {
        return (int)cudaErrorInvalidValue;
    }
    SLLM_LAUNCH_CHECK();
    return 0;
}
