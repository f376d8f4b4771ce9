// Y[M, N] = X[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores of sm_100a:
// TMA (cp.async.bulk.tensor) stages 128-byte-swizzled tiles in shared memory, one thread
// issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 256, K = 16) with the accumulator
// in tensor memory, and four warps drain it with tcgen05.ld.  With SWIGLU the 256 accumulator
// columns are 128 gate and the matching 128 up features, and the epilogue writes
// silu(gate) * up (src/scratch_llm/model.py:236-237 of the reference): the activation costs no
// pass over memory.
//
// The reference's own tcgen05 kernel (csrc/gemm/tcgen05_sm100.cu:222-291) is a single-stage
// skeleton whose instruction descriptor is a placeholder (:123-127) and whose tiles ignore the
// block index (:264-265); this kernel is written from the PTX ISA's descriptor formats instead:
//   instruction descriptor: D = f32 (bits 4-5 = 1), A = B = bf16 (bits 7-9 = 10-12 = 1), both
//     K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28;
//   shared-memory descriptor: start >> 4 (bits 0-13), leading byte offset 1 (16-29, unused by
//     swizzled K-major layouts), stride byte offset 1024 >> 4 between 8-row groups (32-45),
//     version 1 (46-47), layout SWIZZLE_128B = 2 (61-63); a K step of 16 elements advances
//     the start address by 32 bytes inside the 128-byte swizzle atom.
//
// Roles in a CTA of 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer and owner of the
// tensor-memory allocation, warps 2-5 = epilogue (warp w reads the lanes 32*(w%4)..+31 it may
// access).  Persistent CTAs (one per SM) walk output tiles of 128 x 256 through 4 pipeline
// stages of 48 KB; the accumulator is double-buffered in tensor memory so that the epilogue of
// one tile overlaps the products of the next.
//
// The launcher's default is the second kernel of this file, the same product on pairs of SMs
// (cta_group::2, tiles of 256 x 256, six stages of 32 KB per SM): see its comment.
//
// Every mbarrier wait is bounded: after TC_WAIT_LIMIT polls a thread records an error code in
// `g_tc_error`, stops waiting, and the CTA still reaches its end, where the tensor memory is
// freed.  No multicast loads, no peer memory (the pair kernel runs in clusters of two CTAs of
// this GPU and multicasts only its tcgen05.commit arrivals).
#include "tc_common.cuh"

namespace sllm {

constexpr int TM = 128, TN = 256, TK = 64, STAGES = 4;
constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TC_THREADS = 192;
constexpr size_t TC_SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

// Writes 32 consecutive outputs of one row; `n_valid` of them exist.
__device__ __forceinline__ void store_row32(bf16* dst, const float (&o)[32], int n_valid,
                                            bool aligned) {
    // whole groups of 8 as 16-byte stores, the rest one by one
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (aligned && n_valid >= 8 * (i + 1)) {
            uint4 q;
            q.x = pack2(o[8 * i + 0], o[8 * i + 1]);
            q.y = pack2(o[8 * i + 2], o[8 * i + 3]);
            q.z = pack2(o[8 * i + 4], o[8 * i + 5]);
            q.w = pack2(o[8 * i + 6], o[8 * i + 7]);
            reinterpret_cast<uint4*>(dst)[i] = q;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (8 * i + j < n_valid) dst[8 * i + j] = __float2bfloat16_rn(o[8 * i + j]);
        }
    }
}

// Persistent: gridDim.x CTAs walk the output tiles (token blocks fastest, so that consecutive
// tiles share a tile of W, which then streams from HBM once while the smaller activations are
// re-read from L2).  The accumulator is double-buffered in tensor memory (2 x 256 columns):
// the epilogue warps drain tile i while the MMA warp already multiplies tile i + 1.
// SWIGLU: W = [gate rows; up rows] (n_half each); column block j covers features j*128..+127
// and Y has n_half columns.
template <bool SWIGLU>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               bf16* __restrict__ Y, int M, int N, int K, int64_t ldy, int n_half, int tiles_m,
               int tiles_n) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        ((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_stage = smem;                          // STAGES x 16 KB
    unsigned char* b_stage = smem + STAGES * A_BYTES;       // STAGES x 32 KB
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;     // [2]: the MMA warp has finished a tile
    uint64_t* acc_empty = acc_full + 2;      // [2]: the four epilogue warps have drained it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TK - 1) / TK;
    const int total_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TM, n_blk = tile / tiles_m;
                const int w_row0 = SWIGLU ? n_blk * 128 : n_blk * TN;
                const int w_row1 = SWIGLU ? n_half + n_blk * 128 : n_blk * TN + 128;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(a_stage + s * A_BYTES, &map_x, &full[s], kb * TK, m0);
                    tma_load_2d(b_stage + s * B_BYTES, &map_w, &full[s], kb * TK, w_row0);
                    tma_load_2d(b_stage + s * B_BYTES + B_BYTES / 2, &map_w, &full[s], kb * TK,
                                w_row1);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) |
                                   ((uint32_t)(TM >> 4) << 24);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * TN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(smem_u32(a_stage + s * A_BYTES));
                    const uint64_t db = make_smem_desc(smem_u32(b_stage + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k)   // 32 bytes = 2 units of 16 bytes per K step
                        umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(&empty[s]);   // the stage is free once these products have read it
                }
                umma_commit(&acc_full[buf]);  // arrives when every product of the tile is done
            }
        }
    } else {
        const int quad = warp & 3;        // the 32 tensor-memory lanes this warp may read
        uint32_t local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const uint32_t buf = local & 1;
            const int m0 = (tile % tiles_m) * TM, n_blk = tile / tiles_m;
            const int row = m0 + quad * 32 + lane;
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, 3)) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + buf * TN + ((uint32_t)(quad * 32) << 16);
            const bool aligned = (ldy & 7) == 0;
            if (!SWIGLU) {
                const int n0 = n_blk * TN;
#pragma unroll 1
                for (int c = 0; c < TN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + c * 32, v);
                    tmem_ld_wait();
                    const int col = n0 + c * 32;
                    if (row < M && col < N) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]);
                        store_row32(Y + (int64_t)row * ldy + col, o, N - col, aligned);
                    }
                }
            } else {
                constexpr int bn = 128;     // features per tile of this kernel
                const int f0 = n_blk * bn;
#pragma unroll 1
                for (int c = 0; c * 32 < bn; ++c) {
                    uint32_t gv[32], uv[32];
                    tmem_ld32(lane_addr + c * 32, gv);
                    tmem_ld32(lane_addr + bn + c * 32, uv);
                    tmem_ld_wait();
                    const int col = f0 + c * 32;
                    if (row < M && col < n_half) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            // gate and up are rounded to bfloat16 first, as the unfused path does
                            const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gv[i])));
                            const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(uv[i])));
                            o[i] = g / (1.0f + __expf(-g)) * u;
                        }
                        store_row32(Y + (int64_t)row * ldy + col, o, n_half - col, aligned);
                    }
                }
            }
            // this warp has read its part of the buffer: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n"
                     ::"r"(tmem_base), "r"(512u) : "memory");
    }
}


// ------------------------------------------------------------------------------------------
// The same product on PAIRS of SMs (tcgen05 cta_group::2): a cluster of two CTAs owns an output
// tile of 256 tokens x 256 features.  Each CTA stages its own 128 token rows of X and ITS HALF
// of the tile's 256 rows of W (CTA 0 the first 128, CTA 1 the last 128; with SWIGLU the gate
// rows and the up rows), and one thread of CTA 0 issues tcgen05.mma.cta_group::2 with M = 256:
// the tensor cores of both SMs read both halves of W through the cluster's shared memory, so
// every SM fetches 32 KB per K step of 64 instead of 48 KB and six stages fit where four did.
// (The single-SM kernel is bound by what the SMs can fetch from L2, not by its tensor pipe.)
//
// Barriers.  full[s] lives in CTA 0 and counts the bytes of BOTH CTAs' copies (each CTA's TMA
// instruction carries .cta_group::2 and names CTA 0's barrier; no multicast is involved).
// empty[s] and acc_full[b] exist in both CTAs and are signalled in both by one
// tcgen05.commit...multicast::cluster.  acc_empty[b] lives in CTA 0 and collects the eight
// epilogue warps of the pair (the peer's arrive through mapa).  Tensor memory is allocated and
// freed by warp 1 of both CTAs together (cta_group::2); the CTAs leave together (cluster barrier).
constexpr int STAGES2 = 6;
constexpr int B_HALF_BYTES = 128 * TK * 2, STAGE2_BYTES = A_BYTES + B_HALF_BYTES;
constexpr size_t TC2_SMEM = (size_t)STAGES2 * STAGE2_BYTES + 1024 /*align*/ + 256 /*barriers*/;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The barrier at the same shared-memory offset in CTA 0 of the pair.
__device__ __forceinline__ uint32_t leader_addr(const void* local) {
    return smem_u32(local) & 0xFEFFFFFFu;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint32_t leader_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the products issued so
// far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;\n" ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile(
        "{\n.reg .b32 ra;\n"
        "mapa.shared::cluster.u32 ra, %0, 0;\n"
        "mbarrier.arrive.shared::cluster.b64 _, [ra];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cluster_barrier_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// tiles_m counts blocks of 256 tokens here.  gridDim.x = 2 * number of clusters.
// `bn`: rows of W that each CTA of the pair contributes to a tile (the instruction's N is
// 2 * bn; map_w's box has bn rows).  Plain products use 128.  With SWIGLU a tile is bn features
// (CTA 0 brings their gate rows, CTA 1 their up rows), and bn may be any multiple of 16 up to
// 128: the launcher picks the one whose tiles fill the pairs' rounds best.
template <bool SWIGLU>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                bf16* __restrict__ Y, int M, int N, int K, int64_t ldy, int n_half, int tiles_m,
                int tiles_n, int bn) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        ((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_stage = smem;                              // STAGES2 x 16 KB
    unsigned char* b_stage = smem + STAGES2 * A_BYTES;          // STAGES2 x 16 KB (this CTA's half)
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE2_BYTES);
    uint64_t* empty = full + STAGES2;
    uint64_t* acc_full = empty + STAGES2;     // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2], used in CTA 0
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int k_blocks = (K + TK - 1) / TK;
    const int total_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier_all();          // the peer's barriers exist before anything is signalled there
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster; tile < total_tiles && ok; tile += n_clusters) {
                const int m0 = (tile % tiles_m) * (2 * TM) + (int)rank * TM, n_blk = tile / tiles_m;
                const int w_row = SWIGLU ? (rank == 0 ? n_blk * bn : n_half + n_blk * bn)
                                         : n_blk * TN + (int)rank * 128;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES2;
                    ok = mbar_wait(&empty[s], ((it / STAGES2) & 1) ^ 1, 1);
                    if (!ok) break;
                    // CTA 0 announces the bytes of both CTAs
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * (A_BYTES + bn * TK * 2));
                    tma_load_2d_pair(a_stage + s * A_BYTES, &map_x, leader_addr(&full[s]), kb * TK, m0);
                    tma_load_2d_pair(b_stage + s * B_HALF_BYTES, &map_w, leader_addr(&full[s]), kb * TK,
                                     w_row);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   ((uint32_t)((2 * bn) >> 3) << 17) |
                                   ((uint32_t)((2 * TM) >> 4) << 24);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = cluster; tile < total_tiles && ok; tile += n_clusters, ++local) {
                const uint32_t buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * TN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES2;
                    ok = mbar_wait(&full[s], (it / STAGES2) & 1, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(smem_u32(a_stage + s * A_BYTES));
                    const uint64_t db = make_smem_desc(smem_u32(b_stage + s * B_HALF_BYTES));
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k)
                        umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(&empty[s]);   // both CTAs may refill the stage
                }
                umma_commit_pair(&acc_full[buf]);  // both CTAs' epilogue warps may drain
            }
        }
    } else {
        const int quad = warp & 3;
        uint32_t local = 0;
        for (int tile = cluster; tile < total_tiles; tile += n_clusters, ++local) {
            const uint32_t buf = local & 1;
            const int m0 = (tile % tiles_m) * (2 * TM) + (int)rank * TM, n_blk = tile / tiles_m;
            const int row = m0 + quad * 32 + lane;
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, 3)) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + buf * TN + ((uint32_t)(quad * 32) << 16);
            const bool aligned = (ldy & 7) == 0;
            if (!SWIGLU) {
                const int n0 = n_blk * TN;
#pragma unroll 1
                for (int c = 0; c < TN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + c * 32, v);
                    tmem_ld_wait();
                    const int col = n0 + c * 32;
                    if (row < M && col < N) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]);
                        store_row32(Y + (int64_t)row * ldy + col, o, N - col, aligned);
                    }
                }
            } else {
                // gate at columns 0..bn-1 of the buffer, up at bn..2 bn - 1 (a last chunk of 16
                // features reads 16 columns more than it keeps)
                const int f0 = n_blk * bn;
#pragma unroll 1
                for (int c = 0; c * 32 < bn; ++c) {
                    uint32_t gv[32], uv[32];
                    tmem_ld32(lane_addr + c * 32, gv);
                    tmem_ld32(lane_addr + bn + c * 32, uv);
                    tmem_ld_wait();
                    const int col = f0 + c * 32;
                    if (row < M && col < n_half) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            // gate and up are rounded to bfloat16 first, as the unfused path does
                            const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gv[i])));
                            const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(uv[i])));
                            o[i] = g / (1.0f + __expf(-g)) * u;
                        }
                        const int keep = bn - c * 32;    // features of this tile left from col on
                        store_row32(Y + (int64_t)row * ldy + col, o,
                                    n_half - col < keep ? n_half - col : keep, aligned);
                    }
                }
            }
            // this warp has read its part of the buffer: tell the thread that issues the products
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier_all();          // nobody leaves while the pair may still touch its memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n"
                     ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld, boxes of box_rows rows x 64 columns, 128-byte
// swizzle.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int64_t ld,
                     int box_rows = 128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace sllm

using namespace sllm;

static int g_gemm_pairs = 1;
static int g_gemm_tile = 0;
// Features per tile of the pair kernel's fused gate/up product: 0 (default) lets the launcher
// choose, else a multiple of 16 from 16 to 128.
SLLM_EXPORT void sllm_gemm_tc_set_tile(int features) {
    g_gemm_tile = (features >= 16 && features <= 128 && features % 16 == 0) ? features : 0;
}

// The tile width (features) the pair kernel uses for gate/up + SwiGLU of M tokens and n_half
// features on n_pairs SM pairs.  A tile is 256 tokens x bn features and every pair works
// through ceil(tiles / pairs) tiles.  112 instead of 128 is taken where it needs no more
// rounds: every round is then an eighth shorter.  Measured (us, 128 / 112): 14336 features x
// 4096 at 1,024 tokens, 7 rounds either way, 204 / 178; at 512 tokens 120 / 116; 8192 x 2048 at
// 448 tokens 40.7 / 38.0.  Where 112 needs a round more it loses although the rounds are
// shorter (2,048 tokens: 13 rounds of 128 take 329, 14 rounds of 112 take 366), because full
// rounds are bound by what the SMs fetch, and narrower tiles fetch the activations more often;
// widths below 112 lost everywhere.
SLLM_EXPORT int sllm_gemm_tc_swiglu_tile(int M, int n_half, int n_pairs) {
    if (g_gemm_tile) return g_gemm_tile;
    if (M <= 0 || n_half <= 0 || n_pairs <= 0) return 128;
    const int64_t tiles_m = (M + 2 * TM - 1) / (2 * TM);
    const int64_t rounds128 = (tiles_m * ((n_half + 127) / 128) + n_pairs - 1) / n_pairs;
    const int64_t rounds112 = (tiles_m * ((n_half + 111) / 112) + n_pairs - 1) / n_pairs;
    return rounds112 <= rounds128 ? 112 : 128;
}

// 1 (default): tiles of 256 tokens on pairs of SMs (cta_group::2); 0: tiles of 128 tokens on
// single SMs.
SLLM_EXPORT void sllm_gemm_tc_set_pairs(int on) { g_gemm_pairs = on ? 1 : 0; }

// The first error a bounded wait recorded since the last call (0 = none): 1 = producer waiting
// for a free stage, 2 = MMA issuer waiting for data, 3 = epilogue waiting for the accumulator,
// 4 = MMA issuer waiting for a drained accumulator buffer.
// Synchronises the device.
SLLM_EXPORT int sllm_gemm_tc_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return code;
}

// X [M, K], W [N, K] bfloat16, 16-byte aligned with row strides that are multiples of 8;
// Y bfloat16 [M, N] (swiglu = 0) or [M, N / 2] (swiglu = 1, W = [gate rows; up rows]).
SLLM_EXPORT int sllm_gemm_tc(const void* X, const void* W, void* Y, int M, int N, int K,
                             int64_t ldx, int64_t ldw, int64_t ldy, int swiglu,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || (swiglu && (N % 2)))
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)Y & 1))
        return (int)cudaErrorInvalidValue;
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return (int)cudaErrorUnknown;
    }
    const bool pairs = g_gemm_pairs && n_sm >= 2;
    const int n_half = N / 2;
    // rows of W per CTA and tile: 128, or the fused gate/up product's chosen width on pairs
    const int bn = (swiglu && pairs) ? sllm_gemm_tc_swiglu_tile(M, n_half, n_sm / 2) : 128;
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, X, M, K, ldx) || !make_map(&map_w, W, N, K, ldw, bn))
        return (int)cudaErrorNotSupported;
    const int tiles_n = swiglu ? (n_half + bn - 1) / bn : (N + TN - 1) / TN;
    const int tiles_m = (M + TM - 1) / TM;
    if ((int64_t)tiles_m * tiles_n > 0x7fffffff) return (int)cudaErrorInvalidValue;
    if (pairs) {
        // pairs of SMs: tiles of 256 tokens
        const int tiles_m2 = (M + 2 * TM - 1) / (2 * TM);
        const int total2 = tiles_m2 * tiles_n;
        int n_clusters = n_sm / 2;
        if (n_clusters > total2) n_clusters = total2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * n_clusters);
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = TC2_SMEM;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e2;
        if (swiglu) {
            e2 = cudaFuncSetAttribute(gemm_tc2_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC2_SMEM);
            if (e2 != cudaSuccess) return (int)e2;
            e2 = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<true>, map_x, map_w, (bf16*)Y, M, N, K, ldy,
                                    n_half, tiles_m2, tiles_n, bn);
        } else {
            e2 = cudaFuncSetAttribute(gemm_tc2_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC2_SMEM);
            if (e2 != cudaSuccess) return (int)e2;
            e2 = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<false>, map_x, map_w, (bf16*)Y, M, N, K, ldy,
                                    n_half, tiles_m2, tiles_n, 128);
        }
        return (int)e2;
    }
    const int total = tiles_m * tiles_n;
    dim3 grid(total < n_sm ? total : n_sm);
    cudaError_t e;
    if (swiglu) {
        e = cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)TC_SMEM);
        if (e != cudaSuccess) return (int)e;
        gemm_tc_kernel<true><<<grid, TC_THREADS, TC_SMEM, stream>>>(map_x, map_w, (bf16*)Y, M, N, K,
                                                                  ldy, n_half, tiles_m, tiles_n);
    } else {
        e = cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)TC_SMEM);
        if (e != cudaSuccess) return (int)e;
        gemm_tc_kernel<false><<<grid, TC_THREADS, TC_SMEM, stream>>>(map_x, map_w, (bf16*)Y, M, N, K,
                                                                   ldy, n_half, tiles_m, tiles_n);
    }
    SLLM_LAUNCH_CHECK();
    return 0;
}
