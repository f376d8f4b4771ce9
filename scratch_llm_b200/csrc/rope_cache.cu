// Rotary position encoding of q and k (32-bit angles and arithmetic) fused with the write of
// the new keys and values into the paged cache.
//
// Restates src/scratch_llm/model.py:204-220 (rotation of adjacent pairs by the angles of the
// token's absolute position), :284-285 (q and k are rotated, v is not) and the page scatter of
// src/scratch_llm/kv_cache.py:423-428 of the reference.
//
// qkv is [n_tokens, (H + 2G) * hd]: q heads, then k heads, then v heads.  q is rotated in
// place.  k is rotated and stored, v is copied, into
//   pages[page, 0 (K) | 1 (V), g, offset, :]     pages: [n_pages, 2, G, page_size, hd]
// where page = block_table[row, position / page_size], offset = position % page_size.
#include "common.cuh"

namespace sllm {

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_row,
                                     const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, T* __restrict__ pages,
                                     const int* __restrict__ block_table, int table_stride,
                                     int page_size, int H, int G, int hd, int rotate,
                                     int interleaved, int write) {
    pdl_trigger();
    const int64_t n = blockIdx.x;
    const int half = hd >> 1;
    const int pos = positions[n];
    T* row = qkv + n * (int64_t)(H + 2 * G) * hd;
    T* page_base = nullptr;
    int off = 0;
    if (write) {
        const int page = block_table[(int64_t)token_row[n] * table_stride + pos / page_size];
        off = pos % page_size;
        page_base = pages + (int64_t)page * 2 * G * page_size * hd;
    }
    const float* c = cos_t + (int64_t)pos * half;
    const float* s = sin_t + (int64_t)pos * half;
    const int n_rot = (H + G) * half;
    for (int idx = threadIdx.x; idx < n_rot; idx += blockDim.x) {
        const int head = idx / half, j = idx - head * half;
        const int i0 = interleaved ? 2 * j : j;
        const int i1 = interleaved ? 2 * j + 1 : j + half;
        T* h = row + (int64_t)head * hd;
        const float x0 = to_float(h[i0]), x1 = to_float(h[i1]);
        float r0 = x0, r1 = x1;
        if (rotate) {
            const float cj = c[j], sj = s[j];
            r0 = x0 * cj - x1 * sj;
            r1 = x0 * sj + x1 * cj;
        }
        if (head < H) {
            if (rotate) {
                h[i0] = from_float<T>(r0);
                h[i1] = from_float<T>(r1);
            }
        } else if (write) {
            T* dst = page_base + ((int64_t)(head - H) * page_size + off) * hd;
            dst[i0] = from_float<T>(r0);
            dst[i1] = from_float<T>(r1);
        }
    }
    if (write) {
        const T* v = row + (int64_t)(H + G) * hd;
        T* vbase = page_base + (int64_t)G * page_size * hd;
        for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
            const int g = idx / hd, i = idx - g * hd;
            vbase[((int64_t)g * page_size + off) * hd + i] = v[idx];
        }
    }
}

}  // namespace sllm

using namespace sllm;

// rotate = 0 stores k unrotated (a position encoding that is not rotary applies itself first).
SLLM_EXPORT int sllm_rope_kv_write(void* qkv, const int* positions, const int* token_row,
                                   const float* cos_t, const float* sin_t, void* pages,
                                   const int* block_table, int table_stride, int page_size,
                                   int n_tokens, int H, int G, int hd, int rotate,
                                   int interleaved, int write, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || hd <= 0 || (hd & 1) || page_size <= 0) return (int)cudaErrorInvalidValue;
    int threads = 32;
    while (threads < 256 && threads < (H + G) * (hd / 2)) threads <<= 1;
    if (dtype == 0)
        rope_kv_write_kernel<float><<<n_tokens, threads, 0, stream>>>(
            (float*)qkv, positions, token_row, cos_t, sin_t, (float*)pages, block_table,
            table_stride, page_size, H, G, hd, rotate, interleaved, write);
    else if (dtype == 1)
        rope_kv_write_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, positions, token_row, cos_t, sin_t, (__nv_bfloat16*)pages,
            block_table, table_stride, page_size, H, G, hd, rotate, interleaved, write);
    else
        return (int)cudaErrorInvalidValue;
    SLLM_LAUNCH_CHECK();
    return 0;
}
