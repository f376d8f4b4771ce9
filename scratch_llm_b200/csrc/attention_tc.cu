// Causal attention of prompt portions over the paged cache on the tcgen05 tensor cores:
// S = Q K^T and O += P V are tcgen05.mma instructions with S, P and O in tensor memory, keys
// and values arrive page by page through TMA, and the softmax runs with one thread per query
// row (a thread reads its own lane of tensor memory, so row maxima and sums need no shuffles).
//
// Same mathematics as attention_mma.cu (src/scratch_llm/model.py:172-182, :330-345 of the
// reference: scaled scores, causal mask, softmax in 32-bit, probabilities rounded to bfloat16
// before they multiply v, query head h reads kv head h / (H/G)); same packing of a kv head's
// GS = H/G query heads into one tile (packed index p = token * GS + j).
//
//   CTA = 128 packed queries of one (row, kv head), 192 threads:
//     warp 0     TMA producer: the query tile once, then per 128-key tile the pages of K and V
//                (boxes of page_size rows x 64 columns, 128-byte swizzle), 3 stages (1 above head size 128)
//     warp 1     MMA issuer: QK^T (M 128, N 128, K = head size) into S; P V (M 128, N = head
//                size, K 128; A = P from tensor memory, B = V in its stored [key][dim] layout,
//                i.e. MN-major) into O
//     warps 2-5  softmax: S -> registers, mask, running maximum and sum, P -> tensor memory as
//                bfloat16; O is rescaled in tensor memory only when a row's maximum grew by
//                more than 2^8 (the stale reference maximum is exact as long as the final
//                division uses the matching sum); at the end O / l -> global memory
//   tensor memory: two S/P buffers at columns 0..127 and 128..255 (P(t), two bfloat16 per column,
//   takes the place of S(t) in buffer t % 2), O 256..256+HD-1.  While the softmax warps work on
//   S(t) the tensor pipe computes S(t+1), and P(t) V runs beside the softmax of S(t+1).
//
// Takes head sizes that are multiples of 64 up to 256, group sizes that divide 128, page sizes
// that divide 128, no window; other shapes use attention_mma.cu.  What the cache holds beyond
// a row's last position never reaches a result: scores of such keys are overwritten with -inf
// before the softmax, and the rows of V beyond the last position in the row's last key tile
// (the only tile that can hold any) are zeroed in shared memory by the producer warp after
// the copy has landed and before P V is issued, because their probabilities are exactly zero
// and 0 x NaN would be NaN.  Every mbarrier wait is bounded; errors land in g_attn_tc_error.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#error "compile with -DSLLM_HEAD_DIM=<head size>"
#endif

namespace sllm {

typedef __nv_bfloat16 bf16;
constexpr int HD = SLLM_HEAD_DIM;
static_assert(HD % 64 == 0 && HD >= 64 && HD <= 256, "head size: 64, 128, 192 or 256");
constexpr int TQ = 128, TKV = 128, NCB = HD / 64;            // column blocks of 64 (128 bytes)
constexpr int SUB_BYTES = 128 * 128;                          // 128 rows x 128 bytes
constexpr int Q_BYTES = NCB * SUB_BYTES, KV_BYTES = NCB * SUB_BYTES;
constexpr int KV_STAGES = HD <= 128 ? 3 : 1;
// With at least two key/value stages Q K(t+1)^T is issued before P(t) V (two S/P buffers in
// tensor memory take turns); with one stage the next keys arrive only after P(t) V and one
// buffer serves.
constexpr bool EARLY_QK = KV_STAGES >= 2;
constexpr int ATC_THREADS = 192;
constexpr uint32_t SP_COLS = 128, O_COL = 256;   // S/P buffer b at columns 128 b; O behind them
constexpr uint32_t ATC_WAIT_LIMIT = 1u << 24;
constexpr size_t ATC_SMEM = (size_t)Q_BYTES + (size_t)KV_STAGES * 2 * KV_BYTES + 1024 + 256;
constexpr float RESCALE_THRESHOLD = 8.0f;                     // log2 units

__device__ int g_attn_tc_error = 0;

__device__ __forceinline__ float atc_max3(float a, float b, float c) {
    float m;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(m) : "f"(a), "f"(b), "f"(c));
    return m;
}
__device__ __forceinline__ float atc_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// S/P buffer of key tile t and the parity of its use of that buffer's barriers.
__device__ __forceinline__ int atc_buf(int t) { return EARLY_QK ? (t & 1) : 0; }
__device__ __forceinline__ uint32_t atc_phase(int t) { return (uint32_t)((EARLY_QK ? (t >> 1) : t) & 1); }

__device__ __forceinline__ uint32_t atc_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void atc_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(atc_u32(bar)), "r"(count));
}
__device__ __forceinline__ void atc_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n"
                 ::"r"(atc_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void atc_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(atc_u32(bar)) : "memory");
}
__device__ __forceinline__ bool atc_wait(uint64_t* bar, uint32_t parity, int code) {
    const uint32_t addr = atc_u32(bar);
    for (uint32_t i = 0; i < ATC_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (i > 4096) __nanosleep(32);
    }
    atomicCAS(&g_attn_tc_error, 0, code);
    return false;
}
__device__ __forceinline__ void atc_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x,
                                           int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(atc_u32(dst)), "l"(map), "r"(atc_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void atc_tma_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x,
                                           int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(atc_u32(dst)), "l"(map), "r"(atc_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// shared-memory matrix descriptor, 128-byte swizzle: lbo / sbo in bytes
__device__ __forceinline__ uint64_t atc_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void atc_mma_ss(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc,
                                           uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n"
        ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void atc_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t db, uint32_t idesc,
                                           uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n}\n"
        ::"r"(d), "r"(a_tmem), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void atc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(atc_u32(bar)) : "memory");
}
// the load alone; atc_ld_wait() must follow before the values are used
__device__ __forceinline__ void atc_ld32_nowait(uint32_t taddr, float (&r)[32]) {
    uint32_t v[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
          "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
          "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(v[i]);
}
__device__ __forceinline__ void atc_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void atc_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t v[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
          "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
          "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(v[i]);
}
__device__ __forceinline__ void atc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
          "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
          "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
          "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void atc_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void atc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void atc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t atc_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct AtcArgs {
    const int* block_table; int table_stride; int page_size;
    const int* row_start; const int* row_pos0; const int* row_list;
    bf16* out; int64_t out_stride;
    int H, G; float scale_log2;
};

__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
               const AtcArgs a) {
    extern __shared__ unsigned char atc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        ((uintptr_t)atc_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* kv_s = smem + Q_BYTES;                    // stage s: K at s*2*KV_BYTES, V after
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Q_BYTES + (size_t)KV_STAGES * 2 * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;                            // [KV_STAGES]
    uint64_t* kv_empty = kv_full + KV_STAGES;                // [KV_STAGES]
    uint64_t* s_full = kv_empty + KV_STAGES;                 // [2], one per S/P buffer
    uint64_t* p_full = s_full + 2;                           // [2]
    uint64_t* pv_done = p_full + 2;
    uint64_t* o_done = pv_done + 1;                          // the last P V is over
    uint64_t* v_clean = o_done + 1;                          // the last tile's V holds no stale rows
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_clean + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = a.row_list ? a.row_list[blockIdx.y] : blockIdx.y;
    const int g = blockIdx.x;
    const int GS = a.H / a.G;
    const int t0 = a.row_start[r];
    const int n_new = a.row_start[r + 1] - t0;
    const int pos0 = a.row_pos0[r];
    const int n_packed = n_new * GS;
    // Heavy (late) query tiles first, over ALL rows and kv heads: CTAs start in the order of
    // blockIdx.x (kv head), then y (row), then z, so z carries the query tile.  (With the tile
    // in x every kv head's heavy tiles came after the light tiles of the head before, and the
    // last head's heaviest tile, started late, set the end: 64 us instead of 55 at 2,048
    // tokens.)
    const int q_tile = (int)gridDim.z - 1 - (int)blockIdx.z;
    const int q0 = q_tile * TQ;
    if (q0 >= n_packed) return;
    const int tok_first = q0 / GS;
    const int last_pos = pos0 + min(n_packed - 1, q0 + TQ - 1) / GS;
    const int n_tiles = last_pos / TKV + 1;

    if (threadIdx.x == 0) {
        atc_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            atc_init(&kv_full[s], 1);
            atc_init(&kv_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            atc_init(&s_full[b], 1);
            atc_init(&p_full[b], 4);
        }
        atc_init(pv_done, 1);
        atc_init(o_done, 1);
        atc_init(v_clean, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(atc_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    atc_fence_before();
    __syncthreads();
    atc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // The whole warp produces: lane 0 owns the barriers, every lane looks up and copies the
        // pages lane, lane + 32, ... of a tile, so the page lookups of a tile overlap.
        if (lane == 0) {
            // queries: box (64 columns, GS heads, 128 / GS tokens) per 64-column block
            atc_expect_tx(q_full, Q_BYTES);
            for (int c = 0; c < NCB; ++c)
                atc_tma_3d(q_s + c * SUB_BYTES, &map_q, q_full, c * 64, g * GS, t0 + tok_first);
        }
        const int pages_per_tile = TKV / a.page_size;
        const int64_t rows_per_page = (int64_t)2 * a.G * a.page_size;
        const int* table = a.block_table + (int64_t)r * a.table_stride;
        const int n_pages_held = last_pos / a.page_size + 1;
        const int spare = table[0];   // stands in for pages the row does not hold (masked keys)
        bool cleaned = false;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % KV_STAGES;
            // next tile's page numbers are requested before the wait for a free stage
            int my_page[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = lane + 32 * u, lp = t * pages_per_tile + i;
                my_page[u] = (i < pages_per_tile && lp < n_pages_held) ? table[lp] : spare;
                if (my_page[u] < 0) my_page[u] = spare;
            }
            int ok = 1;
            if (lane == 0) {
                ok = atc_wait(&kv_empty[s], ((t / KV_STAGES) & 1) ^ 1, 1) ? 1 : 0;
                if (ok) atc_expect_tx(&kv_full[s], 2 * KV_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            unsigned char* k_dst = kv_s + (size_t)s * 2 * KV_BYTES;
            unsigned char* v_dst = k_dst + KV_BYTES;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = lane + 32 * u;
                if (i >= pages_per_tile) break;
                const int64_t row_k = (int64_t)my_page[u] * rows_per_page + (int64_t)g * a.page_size;
                const int64_t row_v = row_k + (int64_t)a.G * a.page_size;
                for (int c = 0; c < NCB; ++c) {
                    atc_tma_2d(k_dst + c * SUB_BYTES + i * a.page_size * 128, &map_kv, &kv_full[s],
                               c * 64, (int)row_k);
                    atc_tma_2d(v_dst + c * SUB_BYTES + i * a.page_size * 128, &map_kv, &kv_full[s],
                               c * 64, (int)row_v);
                }
            }
            if (t == n_tiles - 1) {
                // Keys beyond last_pos (the rest of the row's last page, pages it does not hold)
                // are whatever earlier requests left there.  Their probabilities are exactly
                // zero, but 0 x NaN is NaN: zero those rows of V (generic-proxy stores), make
                // them visible to the tensor pipe's reads (async proxy), then tell the MMA warp.
                // A key's row is 128 contiguous bytes per 64-column block (the swizzle permutes
                // 16-byte pieces inside a row only).
                if (atc_wait(&kv_full[s], (t / KV_STAGES) & 1, 9)) {
                    const int first_stale = last_pos - t * TKV + 1;      // 1..128
                    const int n16 = (TKV - first_stale) * 8;             // 16-byte pieces per block
                    for (int c = 0; c < NCB; ++c) {
                        uint4* base = reinterpret_cast<uint4*>(v_dst + c * SUB_BYTES +
                                                               first_stale * 128);
                        for (int i = lane; i < n16; i += 32) base[i] = make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
                __syncwarp();
                if (lane == 0) atc_arrive(v_clean);
                cleaned = true;
            }
        }
        // (a producer that gave up still releases the MMA warp, which then meets its own limit)
        if (!cleaned && lane == 0) atc_arrive(v_clean);
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptors: D f32, A and B bf16; QK^T: both K-major, N = 128;
            // P V: B (= V) MN-major, N = head size
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) |
                                      ((uint32_t)(TKV >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);
            bool ok = atc_wait(q_full, 0, 2);
            // the descriptors are built once, so that a product costs this thread an addition
            // (see attn_tc2_kernel)
            uint64_t dq[HD / 16];
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
                dq[kk] = atc_desc(atc_u32(q_s) + (kk / 4) * SUB_BYTES, 16, 1024) + 2 * (kk % 4);
            const uint64_t dk0 = atc_desc(atc_u32(kv_s), 16, 1024);                    // stage 0
            const uint64_t dv0 = atc_desc(atc_u32(kv_s) + KV_BYTES, SUB_BYTES, 1024);
            constexpr uint64_t STAGE_STEP = (2 * KV_BYTES) >> 4;
            // S(t) = Q K(t)^T into the tile's buffer, which the P before it (two tiles back with
            // two buffers, one tile back with one) has left once its P V is done.  A wait on
            // pv_done names the phase by its parity, so the waiter must know that the phase before
            // is over: here the call for the tile before waited for it.
            auto issue_qk = [&](int t) -> bool {
                const int s = t % KV_STAGES;
                if (!atc_wait(&kv_full[s], (t / KV_STAGES) & 1, 3)) return false;
                const int back = EARLY_QK ? 2 : 1;
                if (t >= back && !atc_wait(pv_done, (t - back) & 1, 8)) return false;
                atc_fence_after();
                const uint64_t dk = dk0 + (uint64_t)s * STAGE_STEP;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    atc_mma_ss(tmem + SP_COLS * atc_buf(t), dq[kk],
                               dk + (((kk / 4) * SUB_BYTES) >> 4) + 2 * (kk % 4), idesc_qk, kk > 0);
                atc_commit(&s_full[atc_buf(t)]);
                return true;
            };
            // The tensor pipe's order is QK(0), QK(1), PV(0), QK(2), PV(1), ...: while the softmax
            // warps work on S(t), Q K(t+1)^T already runs, and P(t) V runs beside the softmax of
            // S(t+1).  With one key/value stage the order is QK(t), PV(t), QK(t+1).
            if (ok) ok = issue_qk(0);
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int s = t % KV_STAGES;
                if (EARLY_QK && t + 1 < n_tiles) {
                    ok = issue_qk(t + 1);
                    if (!ok) break;
                }
                // O += P V once the softmax warps have written P: K steps of 16 keys
                ok = atc_wait(&p_full[atc_buf(t)], atc_phase(t), 4);
                if (!ok) break;
                if (t == n_tiles - 1) {       // the producer has zeroed the stale rows of V
                    ok = atc_wait(v_clean, 0, 10);
                    if (!ok) break;
                }
                atc_fence_after();
                // V: rows = keys (128 bytes = 64 dims each), 8-key groups 1024 bytes apart,
                // 64-dim blocks SUB_BYTES apart; 16 keys further = 2048 bytes
                const uint64_t dv = dv0 + (uint64_t)s * STAGE_STEP;
                atc_mma_ts(tmem + O_COL, tmem + SP_COLS * atc_buf(t), dv, idesc_pv, t != 0);
#pragma unroll
                for (int kk = 1; kk < TKV / 16; ++kk)
                    atc_mma_ts(tmem + O_COL, tmem + SP_COLS * atc_buf(t) + kk * 8,
                               dv + kk * (2048 >> 4), idesc_pv, 1);
                atc_commit(&kv_empty[s]);
                atc_commit(pv_done);
                if (!EARLY_QK && t + 1 < n_tiles) ok = issue_qk(t + 1);
            }
            // pv_done runs through a phase per tile and a parity cannot name one of many phases
            // to a warp that arrives late: the end has a barrier of its own
            if (ok) atc_commit(o_done);
        }
    } else {
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                    // packed query within the tile
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        const int p = q0 + row;
        const bool valid = p < n_packed;
        const int tok = valid ? p / GS : 0, j = valid ? p - tok * GS : 0;
        const int qpos = pos0 + tok;
        float m_ref = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            const uint32_t sp_col = SP_COLS * atc_buf(t);    // this tile's S, then its P
            ok = atc_wait(&s_full[atc_buf(t)], atc_phase(t), 5);
            if (!ok) break;
            atc_fence_after();
            const int kt = t * TKV;
            // pass 1: the row's maximum over the tile.  Raw scores: the scale is positive, so it
            // commutes with the maximum and is folded into the exponent below.  Only tiles that
            // reach past the row's own position (or rows that do not exist) need the mask.
            float sv[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) atc_ld32_nowait(lane_base + sp_col + c * 32, sv[c]);
            atc_ld_wait();
            const bool masked = !valid || kt + TKV - 1 > qpos;
            if (masked) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (!valid || kt + c * 32 + i > qpos) sv[c][i] = -INFINITY;
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2)    // the three-input maximum takes two scores at once
                    mx4[(i >> 1) & 3] = atc_max3(mx4[(i >> 1) & 3], sv[c][i], sv[c][i + 1]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;
            // the reference maximum moves only when it must (first keys, or growth beyond 2^8)
            float corr = 1.f;
            if (mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx != -INFINITY)) {
                corr = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
                m_ref = mx;
                l_sum *= corr;
            }
            // O may be rescaled once the previous tile's P V has finished (P(t) takes the place
            // of S(t), which this thread has read, so it waits for nothing).  S(t) exists, so the
            // P V two tiles back is over and the parity names the right phase.
            if (t > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                ok = atc_wait(pv_done, (t - 1) & 1, 6);
                if (!ok) break;
                atc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    float ov[32];
                    atc_ld32(lane_base + O_COL + c * 32, ov);
                    uint32_t w[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(ov[i] * corr);
                    atc_st32(lane_base + O_COL + c * 32, w);
                }
            }
            // pass 2: probabilities p = 2^(s * scale - m_ref) (one fused multiply-add and one
            // exponential each; a masked score is -inf and gives 0), their sum, P as bfloat16
            const float neg_ref = m_ref == -INFINITY ? 0.f : -m_ref;   // all masked: p = 0 anyway
            // (two scores per packed multiply-add and per packed add; the exponential is the
            // bare ex2.approx: its operand is never positive by more than 2^8 and a flushed
            // denormal is a zero probability)
            const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
            const float2 ref2 = make_float2(neg_ref, neg_ref);
            float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t w[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int k0 = c * 64 + 2 * i;           // keys k0, k0 + 1 of the tile
                    const float2 x = __ffma2_rn(make_float2(sv[k0 / 32][k0 % 32],
                                                            sv[(k0 + 1) / 32][(k0 + 1) % 32]),
                                                scale2, ref2);
                    const float2 pr = make_float2(atc_ex2(x.x), atc_ex2(x.y));
                    l2[i & 1] = __fadd2_rn(l2[i & 1], pr);
                    w[i] = atc_pack(pr.x, pr.y);
                }
                atc_st32(lane_base + sp_col + c * 32, w);
            }
            l_sum += (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
            atc_st_wait();
            atc_fence_before();
            __syncwarp();
            if (lane == 0) atc_arrive(&p_full[atc_buf(t)]);
        }
        if (ok && atc_wait(o_done, 0, 7)) {
            atc_fence_after();
            const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
            bf16* dst = a.out + (int64_t)(t0 + tok) * a.out_stride + (int64_t)(g * GS + j) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                float ov[32];
                atc_ld32(lane_base + O_COL + c * 32, ov);
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 q4;
                        q4.x = atc_pack(ov[8 * i + 0] * inv, ov[8 * i + 1] * inv);
                        q4.y = atc_pack(ov[8 * i + 2] * inv, ov[8 * i + 3] * inv);
                        q4.z = atc_pack(ov[8 * i + 4] * inv, ov[8 * i + 5] * inv);
                        q4.w = atc_pack(ov[8 * i + 6] * inv, ov[8 * i + 7] * inv);
                        reinterpret_cast<uint4*>(dst + c * 32)[i] = q4;
                    }
                }
            }
        }
    }
    atc_fence_before();
    __syncthreads();
    if (warp == 1) {
        atc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n"
                     ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// Two query tiles per CTA (head sizes up to 128).  The kernel above leaves the tensor pipe idle
// three quarters of the time: its four softmax warps are one warp per scheduler, each a chain of
// dependent instructions.  Here a CTA owns 256 packed queries, tile A and tile B, which share
// every key/value tile in shared memory (half the traffic per query) and have a softmax
// warpgroup each (warps 2-5 and 6-9), so that two independent chains run per scheduler.
//   tensor memory: S/P of A at columns 0..127, S/P of B at 128..255, O of A at 256.., O of B
//   at 256 + HD.. (exactly the 512 columns at head size 128).
//   tensor pipe order: QK_A(0) QK_B(0) | PV_A(t) QK_A(t+1) PV_B(t) QK_B(t+1) | ...: while the
//   softmax of B(t) runs, the pipe does PV_A(t) and QK_A(t+1), and the other way round.  A
//   tile's S(t+1) takes the place of its P(t): the products of one thread execute in order, so
//   QK_X(t+1), issued after PV_X(t), cannot overtake it.
// Tile A holds the earlier queries, so it needs at most as many key tiles as B; a tile that
// lies beyond the row's queries takes no part.
#if SLLM_HEAD_DIM <= 128
constexpr int KV_STAGES2 = HD <= 64 ? 4 : 2;
constexpr int ATC2_THREADS = 320;
constexpr size_t ATC2_SMEM = (size_t)2 * Q_BYTES + (size_t)KV_STAGES2 * 2 * KV_BYTES + 1024 + 256;

__global__ void __launch_bounds__(ATC2_THREADS, 1)
attn_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                const AtcArgs a) {
    extern __shared__ unsigned char atc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        ((uintptr_t)atc_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;                               // tile A, then tile B
    unsigned char* kv_s = smem + 2 * Q_BYTES;                // stage s: K at s*2*KV_BYTES, V after
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * Q_BYTES +
                                                 (size_t)KV_STAGES2 * 2 * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;                            // [KV_STAGES2]
    uint64_t* kv_empty = kv_full + KV_STAGES2;               // [KV_STAGES2]
    uint64_t* s_full = kv_empty + KV_STAGES2;                // [2], one per query tile
    uint64_t* p_full = s_full + 2;                           // [2]
    uint64_t* pv_done = p_full + 2;                          // [2]
    uint64_t* o_done = pv_done + 2;                          // the last P V of both tiles is over
    uint64_t* v_clean = o_done + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_clean + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = a.row_list ? a.row_list[blockIdx.y] : blockIdx.y;
    const int g = blockIdx.x;
    const int GS = a.H / a.G;
    const int t0 = a.row_start[r];
    const int n_new = a.row_start[r + 1] - t0;
    const int pos0 = a.row_pos0[r];
    const int n_packed = n_new * GS;
    // heavy (late) query tiles first, over all rows and kv heads (see attn_tc_kernel)
    const int pair = (int)gridDim.z - 1 - (int)blockIdx.z;
    const int q0 = pair * 2 * TQ;
    if (q0 >= n_packed) return;
    // per tile: does it exist, its last position, its key tiles
    int n_tiles_x[2], last_pos_x[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int qx = q0 + x * TQ;
        const bool there = qx < n_packed;
        last_pos_x[x] = there ? pos0 + min(n_packed - 1, qx + TQ - 1) / GS : -1;
        n_tiles_x[x] = there ? last_pos_x[x] / TKV + 1 : 0;
    }
    const int n_tiles = max(n_tiles_x[0], n_tiles_x[1]);
    const int last_pos = max(last_pos_x[0], last_pos_x[1]);

    if (threadIdx.x == 0) {
        atc_init(q_full, 1);
        for (int s = 0; s < KV_STAGES2; ++s) {
            atc_init(&kv_full[s], 1);
            atc_init(&kv_empty[s], 1);
        }
        for (int x = 0; x < 2; ++x) {
            atc_init(&s_full[x], 1);
            atc_init(&p_full[x], 4);
            atc_init(&pv_done[x], 1);
        }
        atc_init(o_done, 1);
        atc_init(v_clean, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(atc_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    atc_fence_before();
    __syncthreads();
    atc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // producer, as in the kernel above: lane 0 owns the barriers, every lane copies pages
        if (lane == 0) {
            atc_expect_tx(q_full, 2 * Q_BYTES);
            for (int x = 0; x < 2; ++x)
                for (int c = 0; c < NCB; ++c)
                    atc_tma_3d(q_s + x * Q_BYTES + c * SUB_BYTES, &map_q, q_full, c * 64, g * GS,
                               t0 + (q0 + x * TQ) / GS);
        }
        const int pages_per_tile = TKV / a.page_size;
        const int64_t rows_per_page = (int64_t)2 * a.G * a.page_size;
        const int* table = a.block_table + (int64_t)r * a.table_stride;
        const int n_pages_held = last_pos / a.page_size + 1;
        const int spare = table[0];   // stands in for pages the row does not hold (masked keys)
        bool cleaned = false;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % KV_STAGES2;
            int my_page[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = lane + 32 * u, lp = t * pages_per_tile + i;
                my_page[u] = (i < pages_per_tile && lp < n_pages_held) ? table[lp] : spare;
                if (my_page[u] < 0) my_page[u] = spare;
            }
            int ok = 1;
            if (lane == 0) {
                ok = atc_wait(&kv_empty[s], ((t / KV_STAGES2) & 1) ^ 1, 1) ? 1 : 0;
                if (ok) atc_expect_tx(&kv_full[s], 2 * KV_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            unsigned char* k_dst = kv_s + (size_t)s * 2 * KV_BYTES;
            unsigned char* v_dst = k_dst + KV_BYTES;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = lane + 32 * u;
                if (i >= pages_per_tile) break;
                const int64_t row_k = (int64_t)my_page[u] * rows_per_page + (int64_t)g * a.page_size;
                const int64_t row_v = row_k + (int64_t)a.G * a.page_size;
                for (int c = 0; c < NCB; ++c) {
                    atc_tma_2d(k_dst + c * SUB_BYTES + i * a.page_size * 128, &map_kv, &kv_full[s],
                               c * 64, (int)row_k);
                    atc_tma_2d(v_dst + c * SUB_BYTES + i * a.page_size * 128, &map_kv, &kv_full[s],
                               c * 64, (int)row_v);
                }
            }
            if (t == n_tiles - 1) {
                // stale rows of V beyond the CTA's last position are zeroed (see the kernel above)
                if (atc_wait(&kv_full[s], (t / KV_STAGES2) & 1, 9)) {
                    const int first_stale = last_pos - t * TKV + 1;
                    const int n16 = (TKV - first_stale) * 8;
                    for (int c = 0; c < NCB; ++c) {
                        uint4* base = reinterpret_cast<uint4*>(v_dst + c * SUB_BYTES +
                                                               first_stale * 128);
                        for (int i = lane; i < n16; i += 32) base[i] = make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
                __syncwarp();
                if (lane == 0) atc_arrive(v_clean);
                cleaned = true;
            }
        }
        if (!cleaned && lane == 0) atc_arrive(v_clean);
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) |
                                      ((uint32_t)(TKV >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);
            bool ok = atc_wait(q_full, 0, 2);
            // This one thread feeds the tensor pipe, and a product of 128 x 128 x 16 keeps the
            // pipe busy for about 70 cycles only: whatever the thread computes between two
            // products is time the pipe stands still (with a descriptor built per product the
            // pipe was busy 46 % of the time).  So the descriptors are built once: a product
            // then costs the thread an addition.  (A descriptor's low 14 bits are the
            // shared-memory address / 16, and every address used here lies inside this CTA's
            // allocation, so offsets can be added to the descriptor itself.)
            uint64_t dq[2][HD / 16];
#pragma unroll
            for (int x = 0; x < 2; ++x)
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    dq[x][kk] = atc_desc(atc_u32(q_s + x * Q_BYTES) + (kk / 4) * SUB_BYTES, 16, 1024) +
                                2 * (kk % 4);
            const uint64_t dk0 = atc_desc(atc_u32(kv_s), 16, 1024);                    // stage 0
            const uint64_t dv0 = atc_desc(atc_u32(kv_s) + KV_BYTES, SUB_BYTES, 1024);
            constexpr uint64_t STAGE_STEP = (2 * KV_BYTES) >> 4;
            // S_x(t) = Q_x K(t)^T (the stage's keys must have landed: the caller has waited)
            auto issue_qk = [&](auto xc, int t) {
                constexpr int x = decltype(xc)::value;
                const uint64_t dk = dk0 + (uint64_t)(t % KV_STAGES2) * STAGE_STEP;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    atc_mma_ss(tmem + SP_COLS * x, dq[x][kk],
                               dk + (((kk / 4) * SUB_BYTES) >> 4) + 2 * (kk % 4), idesc_qk, kk > 0);
                atc_commit(&s_full[x]);
            };
            // O_x += P_x(t) V(t)
            auto issue_pv = [&](auto xc, int t) {
                constexpr int x = decltype(xc)::value;
                const uint64_t dv = dv0 + (uint64_t)(t % KV_STAGES2) * STAGE_STEP;
                atc_mma_ts(tmem + O_COL + HD * x, tmem + SP_COLS * x, dv, idesc_pv, t != 0);
#pragma unroll
                for (int kk = 1; kk < TKV / 16; ++kk)
                    atc_mma_ts(tmem + O_COL + HD * x, tmem + SP_COLS * x + kk * 8, dv + kk * (2048 >> 4),
                               idesc_pv, 1);
                atc_commit(&pv_done[x]);
            };
            if (ok) ok = atc_wait(&kv_full[0], 0, 3);
            if (ok) {
                atc_fence_after();
                if (n_tiles_x[0] > 0) issue_qk(std::integral_constant<int, 0>{}, 0);
                if (n_tiles_x[1] > 0) issue_qk(std::integral_constant<int, 1>{}, 0);
            }
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int s = t % KV_STAGES2;
                bool next_ready = false;
                // one query tile's part of step t: P_x(t) V(t), then Q_x K(t+1)^T
                auto tile_step = [&](auto xc) {
                    constexpr int x = decltype(xc)::value;
                    if (t >= n_tiles_x[x]) return;
                    ok = atc_wait(&p_full[x], t & 1, 4);
                    if (!ok) return;
                    if (t == n_tiles - 1) {   // the producer has zeroed the stale rows of V
                        ok = atc_wait(v_clean, 0, 10);
                        if (!ok) return;
                    }
                    atc_fence_after();
                    issue_pv(xc, t);
                    if (t + 1 < n_tiles_x[x]) {
                        if (!next_ready) {
                            ok = atc_wait(&kv_full[(t + 1) % KV_STAGES2], ((t + 1) / KV_STAGES2) & 1, 3);
                            if (!ok) return;
                            atc_fence_after();
                            next_ready = true;
                        }
                        issue_qk(xc, t + 1);
                    }
                };
                tile_step(std::integral_constant<int, 0>{});
                if (ok) tile_step(std::integral_constant<int, 1>{});
                if (!ok) break;
                // every product that reads this stage's keys and values has been issued
                atc_commit(&kv_empty[s]);
            }
            if (ok) atc_commit(o_done);
        }
    } else {
        const int x = warp >= 6 ? 1 : 0;                     // this warpgroup's query tile
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        const uint32_t sp_col = SP_COLS * x, o_col = O_COL + HD * x;
        const int p = q0 + x * TQ + row;
        const bool valid = p < n_packed;
        const int tok = valid ? p / GS : 0, j = valid ? p - tok * GS : 0;
        const int qpos = pos0 + tok;
        const int my_tiles = n_tiles_x[x];
        float m_ref = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int t = 0; t < my_tiles; ++t) {
            ok = atc_wait(&s_full[x], t & 1, 5);
            if (!ok) break;
            atc_fence_after();
            const int kt = t * TKV;
            const bool masked = !valid || kt + TKV - 1 > qpos;
            // pass 1: the row's maximum over the tile, 64 scores at a time (the scores are read
            // from tensor memory again in pass 2: that is cheaper than keeping 128 registers)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float sv[2][32];
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    atc_ld32_nowait(lane_base + sp_col + (2 * h + c) * 32, sv[c]);
                atc_ld_wait();
                if (masked) {
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (!valid || kt + (2 * h + c) * 32 + i > qpos) sv[c][i] = -INFINITY;
                }
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx4[(i >> 1) & 3] = atc_max3(mx4[(i >> 1) & 3], sv[c][i], sv[c][i + 1]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;
            float corr = 1.f;
            if (mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx != -INFINITY)) {
                corr = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
                m_ref = mx;
                l_sum *= corr;
            }
            // O_x may be rescaled once this tile's previous P V has finished; S_x(t) exists, so
            // that product was issued, and its phase is the one the parity names
            if (t > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                ok = atc_wait(&pv_done[x], (t - 1) & 1, 6);
                if (!ok) break;
                atc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    float ov[32];
                    atc_ld32(lane_base + o_col + c * 32, ov);
                    uint32_t w[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(ov[i] * corr);
                    atc_st32(lane_base + o_col + c * 32, w);
                }
            }
            // pass 2: probabilities 2^(s * scale - m_ref), their sum, P as bfloat16 in the place
            // of S (the 64 scores of a half are in registers before its 32 columns of P are
            // written, and P's columns 32 h .. lie inside S's columns 64 h ..)
            const float neg_ref = m_ref == -INFINITY ? 0.f : -m_ref;
            const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
            const float2 ref2 = make_float2(neg_ref, neg_ref);
            float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float sv[2][32];
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    atc_ld32_nowait(lane_base + sp_col + (2 * h + c) * 32, sv[c]);
                atc_ld_wait();
                if (masked) {
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (!valid || kt + (2 * h + c) * 32 + i > qpos) sv[c][i] = -INFINITY;
                }
                uint32_t w[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int k0 = 2 * i;                    // keys 64 h + k0, + 1 of the tile
                    const float2 xx = __ffma2_rn(make_float2(sv[k0 / 32][k0 % 32],
                                                             sv[(k0 + 1) / 32][(k0 + 1) % 32]),
                                                 scale2, ref2);
                    const float2 pr = make_float2(atc_ex2(xx.x), atc_ex2(xx.y));
                    l2[i & 1] = __fadd2_rn(l2[i & 1], pr);
                    w[i] = atc_pack(pr.x, pr.y);
                }
                atc_st32(lane_base + sp_col + h * 32, w);
            }
            l_sum += (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
            atc_st_wait();
            atc_fence_before();
            __syncwarp();
            if (lane == 0) atc_arrive(&p_full[x]);
        }
        if (ok && my_tiles > 0 && atc_wait(o_done, 0, 7)) {
            atc_fence_after();
            const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
            bf16* dst = a.out + (int64_t)(t0 + tok) * a.out_stride + (int64_t)(g * GS + j) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                float ov[32];
                atc_ld32(lane_base + o_col + c * 32, ov);
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 q4;
                        q4.x = atc_pack(ov[8 * i + 0] * inv, ov[8 * i + 1] * inv);
                        q4.y = atc_pack(ov[8 * i + 2] * inv, ov[8 * i + 3] * inv);
                        q4.z = atc_pack(ov[8 * i + 4] * inv, ov[8 * i + 5] * inv);
                        q4.w = atc_pack(ov[8 * i + 6] * inv, ov[8 * i + 7] * inv);
                        reinterpret_cast<uint4*>(dst + c * 32)[i] = q4;
                    }
                }
            }
        }
    }
    atc_fence_before();
    __syncthreads();
    if (warp == 1) {
        atc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n"
                     ::"r"(tmem), "r"(512u) : "memory");
    }
}


#endif  // SLLM_HEAD_DIM <= 128

typedef CUresult (*AtcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtcEncodeFn atc_encode_fn() {
    static AtcEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (AtcEncodeFn)p;
    }
    return fn;
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attn_tc_head_dim() { return HD; }

// Which kernel head sizes up to 128 run.  1 (the default): two query tiles per CTA when the
// launch has at least as many such CTAs as the device has SMs, else one tile per CTA (measured
// at 32 query heads over 8 kv heads, one / two tiles in us: 1,024 tokens = 128 such CTAs 21.9 /
// 27.0, 1,280 tokens = 160 CTAs 31.8 / 31.5, 2,048 tokens 58.2 / 51.8, 4,096 tokens 175 / 159);
// 2: always two tiles; 0: always one (head sizes above 128 have that kernel only).
static int g_atc_two_tiles = 1;
SLLM_EXPORT void sllm_attn_tc_set_two_tiles(int mode) {
    g_atc_two_tiles = mode < 0 ? 0 : (mode > 2 ? 2 : mode);
}

// 1 if this kernel takes the shape, 0 if attention_mma.cu must serve it.
SLLM_EXPORT int sllm_attn_tc_supports(int H, int G, int page_size, int window) {
    if (H <= 0 || G <= 0 || H % G) return 0;
    const int GS = H / G;
    return (128 % GS == 0) && page_size > 0 && (128 % page_size == 0) && window == 0;
}

SLLM_EXPORT int sllm_attn_tc_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return code;
}

// q / out: [n_tokens, stride] bfloat16, head h at columns [h*HD, (h+1)*HD).  pages:
// [n_pages, 2, G, page_size, HD] bfloat16 (places no listed row uses may hold anything).  row_list: the n_list rows served
// (nullptr: rows 0..n_list-1); max_new: the largest number of new tokens among them.
SLLM_EXPORT int sllm_attn_tc(const void* q, int64_t q_stride, int64_t n_tokens, const void* pages,
                             int64_t n_pages, const int* block_table, int table_stride,
                             int page_size, const int* row_start, const int* row_pos0,
                             const int* row_list, int n_list, int max_new, void* out,
                             int64_t out_stride, int H, int G, float scale, cudaStream_t stream) {
    if (n_list <= 0 || max_new <= 0) return 0;
    if (!sllm_attn_tc_supports(H, G, page_size, 0) || n_list > 65535 || G > 65535 ||
        (q_stride % 8) || (out_stride % 8) || ((uintptr_t)q & 15) || ((uintptr_t)pages & 15) ||
        ((uintptr_t)out & 15))
        return (int)cudaErrorInvalidValue;
    if (n_pages * 2 * G * page_size > 0x7fffffffLL || n_tokens > 0x7fffffffLL)
        return (int)cudaErrorInvalidValue;
    // the query tiles of a row are the grid's z: at most 65,535 of them
    if (((int64_t)max_new * (H / G) + TQ - 1) / TQ > 65535) return (int)cudaErrorInvalidValue;
    AtcEncodeFn fn = atc_encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const int GS = H / G;
    CUtensorMap map_q, map_kv;
    {   // q as (column, head, token)
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
        cuuint32_t box[3] = {64u, (cuuint32_t)GS, (cuuint32_t)(TQ / GS)};
        cuuint32_t elem[3] = {1u, 1u, 1u};
        if (fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    {   // the cache as rows of HD columns: row = ((page * 2 + kv) * G + g) * page_size + offset
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)(n_pages * 2 * G * page_size)};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64u, (cuuint32_t)page_size};
        cuuint32_t elem[2] = {1u, 1u};
        if (fn(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims,
               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    AtcArgs a;
    a.block_table = block_table; a.table_stride = table_stride; a.page_size = page_size;
    a.row_start = row_start; a.row_pos0 = row_pos0; a.row_list = row_list;
    a.out = (bf16*)out; a.out_stride = out_stride; a.H = H; a.G = G;
    a.scale_log2 = scale * 1.4426950408889634f;
    cudaError_t e;
#if SLLM_HEAD_DIM <= 128
    // Two query tiles per CTA halve the number of CTAs: that pays once the launch still fills
    // the device several times over (measured at 32 heads over 8 kv heads of size 128: 600
    // against 655 us at 8,192 tokens, but 186 against 177 us at 4,096 and 70.6 against 64.3 us
    // at 2,048, where two and four rounds of CTAs are left).
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n_sm = 148;
    }
    const int64_t pair_ctas = (((int64_t)max_new * GS + 2 * TQ - 1) / (2 * TQ)) * n_list * G;
    if (g_atc_two_tiles == 1 ? pair_ctas >= (int64_t)n_sm : g_atc_two_tiles == 2) {
        e = cudaFuncSetAttribute(attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ATC2_SMEM);
        if (e != cudaSuccess) return (int)e;
        dim3 grid2(G, n_list, ((int64_t)max_new * GS + 2 * TQ - 1) / (2 * TQ));
        attn_tc2_kernel<<<grid2, ATC2_THREADS, ATC2_SMEM, stream>>>(map_q, map_kv, a);
        SLLM_LAUNCH_CHECK();
        return 0;
    }
#endif
    e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)ATC_SMEM);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(G, n_list, ((int64_t)max_new * GS + TQ - 1) / TQ);
    attn_tc_kernel<<<grid, ATC_THREADS, ATC_SMEM, stream>>>(map_q, map_kv, a);
    SLLM_LAUNCH_CHECK();
    return 0;
}
