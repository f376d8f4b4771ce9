// The pieces that the persistent small-batch products share (gemv_tma.cu: one product per
// launch; gemv_chain.cu: several products that feed one another in one launch): sizes of the
// shared-memory pipeline, bounded mbarrier waits, the tensor copy of a stage, the exchange of
// partial sums through (value, flag) words, and the m16n8k16 product with the tokens as m.
// Each library that includes this has its own error word `g_gemv_error`.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace sllm {

typedef __nv_bfloat16 bf16;
constexpr int GT_ROWS = 8;                       // W rows of a unit (the n of m16n8k16)
#ifndef GT_KS_DEF
#define GT_KS_DEF 512
#endif
constexpr int GT_KS = GT_KS_DEF;                 // k of a stage
constexpr int GT_MIN_SPLITS = 2;                 // ranges of K: at least this many, and more
constexpr int GT_MAX_RANGE = 4096;               // for a long K, so that no range exceeds this
constexpr int GT_MAX_SPLITS = 64;
constexpr int GT_SMEM_LIMIT = 232448 - 1024;     // one CTA per SM; 1024 bytes go to alignment
constexpr int GT_CWARPS = 8;                     // consumer warps
constexpr int GT_FWARPS = 4;                     // combiner warps launched
constexpr int GT_RED_BYTES = 16384;              // hand-over slots between consumers and combiners
constexpr int GT_PWARPS = 1;                     // producer warps (eight lanes issue the copies)
constexpr int GT_THREADS = 32 * (GT_CWARPS + GT_PWARPS + GT_FWARPS);
constexpr int GT_BLOCK_BYTES = GT_ROWS * GT_KS * 2;   // 8 rows of a stage: [k / 64][row][128 bytes], swizzled
constexpr int GT_TOK = 8;                        // tokens of the product
constexpr int GT_VPL = GT_ROWS * GT_TOK / 32;    // values of a tile per lane of a combiner warp
constexpr uint32_t GT_WAIT_LIMIT = 1u << 24;
constexpr int GT_MAX_STAGES = 48;

static __device__ int g_gemv_error = 0;

__device__ __forceinline__ uint32_t gt_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void gt_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(gt_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void gt_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n"
                 ::"r"(gt_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gt_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(gt_smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false = gave up after about two seconds
// (error recorded).  A waiter must be at most one phase away from the barrier's current phase:
// the parity cannot tell phases apart that are two apart.
__device__ __forceinline__ bool gt_mbar_wait(uint64_t* bar, uint32_t parity, int code) {
    const uint32_t addr = gt_smem_u32(bar);
    uint64_t t0 = 0;
    for (uint32_t i = 0; i < GT_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 255) == 255) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) break;
            __nanosleep(64);
        }
    }
    atomicCAS(&g_gemv_error, 0, code);
    return false;
}
// One box of 16 rows x GT_KS columns of W: global -> shared through the tensor map (128-byte
// swizzle), completion counted in bytes on `bar`.  c1 = first row, c2 = first 64-column chunk.
__device__ __forceinline__ void gt_tma_load(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(gt_smem_u32(smem_dst)), "l"(map), "r"(gt_smem_u32(bar)), "r"(0), "r"(c1), "r"(c2)
        : "memory");
}
// Takes the N words words[0], words[32], ... of a range: loads them all at once, again until
// every flag is set (for about two seconds at most), puts them back to zero and returns the
// values.
template <int N>
__device__ __forceinline__ void gt_take_words(float2* words, float* value) {
    uint64_t t0 = 0;
    bool all = false;
    for (uint32_t i = 0; i < GT_WAIT_LIMIT && !all; ++i) {
        uint32_t flags = 1;
#pragma unroll
        for (int n = 0; n < N; ++n) {
            uint32_t flag;
            asm volatile("ld.volatile.global.v2.b32 {%0, %1}, [%2];\n"
                         : "=f"(value[n]), "=r"(flag) : "l"(words + 32 * n) : "memory");
            flags &= flag;
        }
        all = flags != 0;
        if (!all && (i & 63) == 63) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) break;
        }
    }
    if (!all) atomicCAS(&g_gemv_error, 0, 5);
#pragma unroll
    for (int n = 0; n < N; ++n) __stcg(words + 32 * n, make_float2(0.f, 0.f));
}
__device__ __forceinline__ void gt_ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(gt_smem_u32(p)));
}
// d += A * B with A = [tokens 0-7; zeros] (a0: k 0-7, a2: k 8-15 of the k-step) and B = 8 rows of W.
__device__ __forceinline__ void gt_mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gt_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

template <typename T> __device__ __forceinline__ void gt_store(T* p, float v);
template <> __device__ __forceinline__ void gt_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void gt_store<bf16>(bf16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

}  // namespace sllm
