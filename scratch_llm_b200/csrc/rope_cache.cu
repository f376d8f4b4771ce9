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
// A token whose row is -1 is padding: it is neither rotated nor stored.
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
    if (token_row[n] < 0) return;   // a padding token: it belongs to no row
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


// The same for bfloat16 with 16-byte accesses: a thread takes 8 consecutive elements of a head
// (adjacent pairing: 4 pairs) or 8 elements of each half (split pairing: 8 pairs).  Arithmetic
// and rounding are those of the kernel above.  hd % 16 == 0.
__device__ __forceinline__ void rotate8(const uint4& a, const uint4& b, const float* c,
                                        const float* s, uint4& ra, uint4& rb) {
    // a holds x0 of 8 pairs, b holds x1 of the same pairs
    const __nv_bfloat16* xa = reinterpret_cast<const __nv_bfloat16*>(&a);
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(&b);
    __nv_bfloat16* ya = reinterpret_cast<__nv_bfloat16*>(&ra);
    __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(&rb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x0 = __bfloat162float(xa[i]), x1 = __bfloat162float(xb[i]);
        ya[i] = __float2bfloat16_rn(x0 * c[i] - x1 * s[i]);
        yb[i] = __float2bfloat16_rn(x0 * s[i] + x1 * c[i]);
    }
}

constexpr int ROPE_HEAD_GROUPS = 4;   // threads that share a token's heads between them

// A thread takes one 8-element unit (adjacent pairing) or one pair of units (split pairing) of
// a token and walks a quarter of the token's heads with it: the angles are fetched once and
// serve every head.
__global__ void rope_kv_write_vec_kernel(__nv_bfloat16* __restrict__ qkv,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ token_row,
                                         const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t,
                                         __nv_bfloat16* __restrict__ pages,
                                         const int* __restrict__ block_table, int table_stride,
                                         int page_size, int H, int G, int hd, int rotate,
                                         int interleaved, int write, int64_t n_items) {
    pdl_wait();
    pdl_trigger();
    typedef __nv_bfloat16 bf16;
    const int half = hd >> 1;
    const int per_head = interleaved ? hd / 8 : hd / 16;   // units of a head
    const int n_heads = write ? H + 2 * G : H;
    const int heads_per_group = (n_heads + ROPE_HEAD_GROUPS - 1) / ROPE_HEAD_GROUPS;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_items;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int u = (int)(i % per_head);
        const int64_t t = i / per_head;
        const int group = (int)(t % ROPE_HEAD_GROUPS);
        const int64_t n = t / ROPE_HEAD_GROUPS;
        const int row = token_row[n];
        if (row < 0) continue;   // a padding token: it belongs to no row
        const int pos = positions[n];
        // first and second group of 8 elements this thread owns in every head
        const int e0 = 8 * u, e1 = half + 8 * u;   // (e1 only with the split pairing)
        float c[8], sn[8];
        if (rotate) {
            const float* cp = cos_t + (int64_t)pos * half + (interleaved ? 4 * u : 8 * u);
            const float* sp = sin_t + (int64_t)pos * half + (interleaved ? 4 * u : 8 * u);
            *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp);
            *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sp);
            if (!interleaved) {
                *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 4);
                *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sp + 4);
            }
        }
        int64_t page_base = 0;
        if (write) {
            const int page = block_table[(int64_t)row * table_stride + pos / page_size];
            page_base = (int64_t)page * 2 * G * page_size * hd + (int64_t)(pos % page_size) * hd;
        }
        bf16* tok = qkv + n * (int64_t)(H + 2 * G) * hd;
        const int head_end = min(n_heads, (group + 1) * heads_per_group);
#pragma unroll 4
        for (int head = group * heads_per_group; head < head_end; ++head) {
            bf16* h = tok + (int64_t)head * hd;
            uint4 a = *reinterpret_cast<const uint4*>(h + e0), b;
            if (!interleaved) b = *reinterpret_cast<const uint4*>(h + e1);
            const bool is_v = head >= H + G;
            if (rotate && !is_v) {
                if (interleaved) {
                    // 4 adjacent pairs inside one group of 8
                    bf16* x = reinterpret_cast<bf16*>(&a);
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float x0 = __bfloat162float(x[2 * p]), x1 = __bfloat162float(x[2 * p + 1]);
                        x[2 * p] = __float2bfloat16_rn(x0 * c[p] - x1 * sn[p]);
                        x[2 * p + 1] = __float2bfloat16_rn(x0 * sn[p] + x1 * c[p]);
                    }
                } else {
                    uint4 ra, rb;
                    rotate8(a, b, c, sn, ra, rb);
                    a = ra;
                    b = rb;
                }
            }
            if (head < H) {
                if (rotate) {
                    *reinterpret_cast<uint4*>(h + e0) = a;
                    if (!interleaved) *reinterpret_cast<uint4*>(h + e1) = b;
                }
                continue;
            }
            const int g = head - H - (is_v ? G : 0);
            bf16* dst = pages + page_base + ((int64_t)(is_v ? G : 0) + g) * page_size * hd;
            *reinterpret_cast<uint4*>(dst + e0) = a;
            if (!interleaved) *reinterpret_cast<uint4*>(dst + e1) = b;
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
    if (dtype == 1 && hd % 16 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)pages & 15) &&
        (!rotate || (!((uintptr_t)cos_t & 15) && !((uintptr_t)sin_t & 15)))) {
        const int64_t n_units = (int64_t)n_tokens * ROPE_HEAD_GROUPS * (interleaved ? hd / 8 : hd / 16);
        int64_t blocks = (n_units + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        return (int)sllm_launch_pdl(rope_kv_write_vec_kernel, dim3((unsigned)blocks), dim3(256), 0,
                                    stream, (__nv_bfloat16*)qkv, positions, token_row, cos_t, sin_t,
                                    (__nv_bfloat16*)pages, block_table, table_stride, page_size, H,
                                    G, hd, rotate, interleaved, write, n_units);
    }
    if (dtype == 1)
        return (int)sllm_launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), 0,
                                    stream, (__nv_bfloat16*)qkv, positions, token_row, cos_t, sin_t,
                                    (__nv_bfloat16*)pages, block_table, table_stride, page_size, H,
                                    G, hd, rotate, interleaved, write, heads_per_block);
    return (int)cudaErrorInvalidValue;
}
