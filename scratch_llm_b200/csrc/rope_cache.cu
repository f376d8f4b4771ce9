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

// grid (tokens, blocks of heads); a block of 256 threads takes as many heads as fit, one thread
// per rotated pair (for v heads: per copied pair).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_row,
                                     const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, T* __restrict__ pages,
                                     const int* __restrict__ block_table, int table_stride,
                                     int page_size, int H, int G, int hd, int rotate,
                                     int interleaved, int write, int heads_per_block) {
    pdl_wait();
    pdl_trigger();
    const int64_t n = blockIdx.x;
    const int half = hd >> 1;
    const int local = threadIdx.x / half, j = threadIdx.x - local * half;
    const int head = blockIdx.y * heads_per_block + local;
    if (local >= heads_per_block || head >= H + 2 * G) return;
    if (head >= H && !write) return;
    const int pos = positions[n];
    T* h = qkv + n * (int64_t)(H + 2 * G) * hd + (int64_t)head * hd;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? 2 * j + 1 : j + half;
    float r0 = to_float(h[i0]), r1 = to_float(h[i1]);
    if (rotate && head < H + G) {
        const float cj = cos_t[(int64_t)pos * half + j], sj = sin_t[(int64_t)pos * half + j];
        const float x0 = r0, x1 = r1;
        r0 = x0 * cj - x1 * sj;
        r1 = x0 * sj + x1 * cj;
    }
    if (head < H) {
        if (rotate) {
            h[i0] = from_float<T>(r0);
            h[i1] = from_float<T>(r1);
        }
        return;
    }
    const int page = block_table[(int64_t)token_row[n] * table_stride + pos / page_size];
    const int off = pos % page_size;
    const bool is_v = head >= H + G;
    const int g = head - H - (is_v ? G : 0);
    T* dst = pages + (((int64_t)page * 2 + (is_v ? 1 : 0)) * G + g) * page_size * hd +
             (int64_t)off * hd;
    if (is_v) {   // v is copied as it is
        dst[i0] = h[i0];
        dst[i1] = h[i1];
    } else {
        dst[i0] = from_float<T>(r0);
        dst[i1] = from_float<T>(r1);
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
    if (hd / 2 > 256) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const int heads_per_block = threads / (hd / 2);
    const int n_heads = write ? H + 2 * G : H;
    dim3 grid(n_tokens, (n_heads + heads_per_block - 1) / heads_per_block);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == 0)
        return (int)sllm_launch_pdl(rope_kv_write_kernel<float>, grid, dim3(threads), 0, stream,
                                    (float*)qkv, positions, token_row, cos_t, sin_t, (float*)pages,
                                    block_table, table_stride, page_size, H, G, hd, rotate,
                                    interleaved, write, heads_per_block);
    if (dtype == 1)
        return (int)sllm_launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), 0,
                                    stream, (__nv_bfloat16*)qkv, positions, token_row, cos_t, sin_t,
                                    (__nv_bfloat16*)pages, block_table, table_stride, page_size, H,
                                    G, hd, rotate, interleaved, write, heads_per_block);
    return (int)cudaErrorInvalidValue;
}
