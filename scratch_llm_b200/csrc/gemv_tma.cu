// Y[M, N] = X[M, K] * W[N, K]^T for up to 8 tokens by a persistent kernel that streams W through
// shared memory with TMA tensor copies: the decode step's matrix products at the sizes of a real
// model, where what counts is that weight bytes are in flight on every SM from the kernel's first
// cycle to its last.
//
// `y = x @ W.T`, weight stored (out, in): src/scratch_llm/model.py:125-133 of the reference; with
// SWIGLU, silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu] (src/scratch_llm/model.py:236-237).  The
// reference's persistent GEMV (csrc/persistent/persistent_gemv_sm90.cu) is a stub; this kernel
// is what that file names: one CTA per SM that lives for the whole product.
//
// Work.  The product is cut into units of 8 rows of W (with SWIGLU: 8 gate rows and the 8 up rows
// that pair with them) times one of S ranges of K (S = 2, more for a long K; 1 for a matrix so
// wide that its row tiles alone spread evenly).  CTA c takes range c % S and the row tiles c / S,
// c / S + grid / S, ...: its slice of the activations is loaded into shared memory once, and
// the units are small enough that 148 CTAs get equal shares.  A unit is streamed in stages of
// 8 rows x 512 columns; every row piece is 1 KB of consecutive memory (with 512-byte pieces
// the DRAM pages were opened twice and the kernel stayed at 5 TB/s).
//
// Roles in a CTA of 13 warps.
//   producer (warp 8): lane l of 8 feeds the ring slots l, l + 8, ...: it waits for the slot to
//     be empty, announces the bytes to the slot's mbarrier and issues one cp.async.bulk.tensor
//     (3-D map: 64 columns, rows, 64-column chunks; 128-byte swizzle) per 8 rows.  The lanes run
//     ahead of the consumers by the whole ring (up to 190 KB), across unit boundaries, and start
//     before the previous kernel of the stream has finished (weights are written by nobody).
//   consumers (warps 0-7): warp w takes the stages w, w + 8, ... whole, so that a barrier is
//     touched by one warp per stage and eight stages are worked on at once.  m16n8k16 with the
//     tokens as m (rows 8-15 are zero registers) and the 8 rows of W as n; the operands come from
//     shared memory by ldmatrix, free of bank conflicts thanks to the swizzle.  At a unit's end
//     every warp hands its partial sums to a combiner warp through shared memory.
//   combiners (warps 9-12): add the eight warps' sums in warp order, then combine the S ranges
//     of the tile through global memory without fences or atomics: a partial sum travels as an
//     8-byte word (value, flag).  The CTA of the last range polls the words of the ranges before
//     it, adds them in the order of the ranges, writes the output and puts the words back to
//     zero.  Nothing depends on timing or on M, so a token's result is bitwise the same at any
//     batch size.  Several units are in flight in the combiners while the consumers go on.
//
// Waiting on CTAs of the same grid: the collecting CTA polls words that CTAs with smaller block
// indices write.  Those CTAs never wait for the collecting one, the grid has at most one CTA per
// SM, and a CTA needs no more than an SM can give: so whatever order the hardware starts the
// CTAs in (usually that of their indices, which keeps the wait short), and also when the
// previous kernel of the stream still holds SMs at this grid's programmatic start, every CTA
// gets its SM without anything of this grid having to finish first, and the wait ends.
//
// Every wait (mbarrier or flag) is bounded: after about two seconds the thread records a code
// in `g_gemv_error` and goes on without waiting (the host reads the word and raises): 1 =
// producer waiting for a free slot, 2 = consumer waiting for data, 3 = consumer waiting for a
// hand-over slot, 4 = combiner waiting for the consumers, 5 = combiner waiting for another range.
#include "gemv_pipe.cuh"

namespace sllm {

struct GemvTmaArgs {
    const bf16* X;
    const bf16* W;
    void* Y;
    float2* partials;     // [tiles][splits - 1][NW * 128] words (value, flag), zero between launches
    int M, N, K;
    int64_t ldx, ldw, ldy;
    int splits;           // ranges of K
    int stages;           // ring depth
    int x_stride;         // elements between token rows of the activations in shared memory
    int ring_offset;      // bytes from the start of shared memory to the ring
    // A product that STARTS a branch of a pre-norm layer may take activations whose RMS norm is
    // not finished: X = stream * gain, and every output of token t still has to be multiplied by
    // rsqrt(sum_p ss_in[p][t] * ss_inv_dim + ss_eps), the factor that is one number per token
    // and so commutes with the product.  ss_in = nullptr: X is what it is.
    const float* ss_in;   // [ss_parts][8]: shares of the tokens' sums of squares
    int ss_parts;
    float ss_inv_dim, ss_eps;
    // A product that ENDS a branch (not with SWIGLU) may put its output into the 32-bit residual
    // stream itself and prepare the next norm: with r = resid[t][f] + round_bf16(y[t][f]),
    //   resid[t][f] = r,   x_out[t][f] = bf16(r * gain[f]),   ss_out[tile][t] = sum_f r^2
    // over the tile's 8 features.  resid = nullptr: Y is stored.
    float* resid;
    int64_t ld_resid;
    const float* gain;
    bf16* x_out;
    int64_t ld_xout;
    float* ss_out;        // [row tiles][8]
};

// Shared memory: [barriers] | the warps' partial sums | activations | ring
template <bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(GT_THREADS, 1) gemv_tma_kernel(const __grid_constant__ CUtensorMap map_w, const GemvTmaArgs a) {
    constexpr int NW = SWIGLU ? 2 : 1;
    constexpr int STAGE_BYTES = NW * GT_BLOCK_BYTES;
    constexpr int TILE_VALUES = NW * GT_ROWS * GT_TOK;
    // combiner warps in use: each has a hand-over slot of its own (8 warps' partial sums), so
    // that it meets the phases of its barriers one after the other
    constexpr int F_FIT = GT_RED_BYTES / (GT_CWARPS * TILE_VALUES * 4);
    constexpr int F = F_FIT < GT_FWARPS ? F_FIT : GT_FWARPS;
    static_assert(F >= 1, "hand-over slots");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the swizzled stages want 1024-byte alignment: the launcher asks for 1024 bytes more
    unsigned char* smem = smem_raw + ((1024u - (gt_smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GT_MAX_STAGES;
    uint64_t* red_full = empty + GT_MAX_STAGES;
    uint64_t* red_empty = red_full + GT_FWARPS;
    float* red = reinterpret_cast<float*>(smem + 1024);      // [F][8 warps][TILE_VALUES]
    bf16* xs = reinterpret_cast<bf16*>(smem + 1024 + GT_RED_BYTES);
    unsigned char* ring = smem + a.ring_offset;              // 1024-byte aligned

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int stages = a.stages;
    const int n_out = SWIGLU ? a.N / 2 : a.N;
    const int tiles = (n_out + GT_ROWS - 1) / GT_ROWS;
    const int S = a.splits;
    const int split = blockIdx.x % S;
    const int tile0 = blockIdx.x / S, tile_step = gridDim.x / S;
    const int total_stages = a.K / GT_KS;
    const int st_begin = (int)((int64_t)split * total_stages / S);
    const int st_end = (int)((int64_t)(split + 1) * total_stages / S);
    const int n_st = st_end - st_begin;           // stages of a unit of this CTA

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            gt_mbar_init(full + s, 1);
            gt_mbar_init(empty + s, 1);
        }
        for (int s = 0; s < F; ++s) {
            gt_mbar_init(red_full + s, GT_CWARPS);
            gt_mbar_init(red_empty + s, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    if (tile0 >= tiles) return;

    if (warp == GT_CWARPS) {
        // ---- producer: lane l (of 8) feeds the slots l, l + 8, ... of the ring, that is, the
        // stages consumer warp l takes.  One lane alone would need about 0.2 us a stage for its
        // chain of wait, announcement and copy; eight lanes run eight such chains side by side.
        // A lane never waits for a slot whose earlier contents were requested in the same round,
        // because the ring has at least 8 slots. ----
        if (lane < GT_CWARPS) {
            int n_units = 0;
            for (int tile = tile0; tile < tiles; tile += tile_step) ++n_units;
            int unit = 0, st = lane;               // stage `st` of unit `unit` is this lane's next
            while (st >= n_st && unit < n_units) { st -= n_st; ++unit; }
            int slot = lane;                        // its slot, and how often the ring has wrapped
            uint32_t wraps = 0;
            bool waited = false;
            while (unit < n_units) {
                if (wraps > 0) {
                    if (!waited) {
                        // the ring is full of weights requested ahead of the previous kernel's
                        // end; from here on the stages are recycled
                        pdl_wait();
                        pdl_trigger();
                        waited = true;
                    }
                    gt_mbar_wait(empty + slot, (wraps - 1) & 1, 1);
                }
                unsigned char* dst = ring + (size_t)slot * STAGE_BYTES;
                gt_mbar_expect_tx(full + slot, STAGE_BYTES);
                const int n0 = (tile0 + unit * tile_step) * GT_ROWS;
                const int chunk = (st_begin + st) * (GT_KS / 64);
                gt_tma_load(dst, &map_w, full + slot, n0, chunk);
                if (SWIGLU) gt_tma_load(dst + GT_BLOCK_BYTES, &map_w, full + slot, n_out + n0, chunk);
                st += GT_CWARPS;
                while (st >= n_st && unit < n_units) { st -= n_st; ++unit; }
                slot += GT_CWARPS;
                if (slot >= stages) { slot -= stages; ++wraps; }
            }
            if (!waited) {
                pdl_wait();
                pdl_trigger();
            }
        }
        return;
    }

    if (warp >= GT_CWARPS + GT_PWARPS) {
        // ---- combiners: warp f takes the units f, f + F, ...; several units are in
        // flight at once, so the latency of the exchange through global memory is off the
        // consumers' path ----
        pdl_wait();
        pdl_trigger();
        const int f = warp - GT_CWARPS - GT_PWARPS;
        // (the barrier page has room left behind its 104 barriers: 32 + 8 floats)
        float* ss_share = reinterpret_cast<float*>(smem + 832);      // [4 warps][8 tokens]
        float* inv_rms = ss_share + GT_FWARPS * GT_TOK;              // [8 tokens]
        if (a.ss_in != nullptr && split == S - 1) {
            // the tokens' factors: the shares are added in a fixed tree (16 strided sums, four
            // of them per warp combined by shuffles, then the warps in order), so the factor
            // does not depend on timing or on the batch
            const int tok = lane & (GT_TOK - 1), sub = f * 4 + (lane >> 3);
            float part = 0.f;
            for (int p = sub; p < a.ss_parts; p += 16) part += __ldcg(a.ss_in + (size_t)p * GT_TOK + tok);
            part += __shfl_xor_sync(0xffffffffu, part, 8);
            part += __shfl_xor_sync(0xffffffffu, part, 16);
            if (lane < GT_TOK) ss_share[f * GT_TOK + lane] = part;
            gt_bar_sync(2, GT_FWARPS * 32);
            if (f == 0 && lane < GT_TOK) {
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < GT_FWARPS; ++i) sum += ss_share[i * GT_TOK + lane];
                inv_rms[lane] = rsqrtf(sum * a.ss_inv_dim + a.ss_eps);
            }
            gt_bar_sync(2, GT_FWARPS * 32);
        }
        if (f >= F) return;
        int round = 0;
        for (int tile = tile0 + f * tile_step; tile < tiles; tile += F * tile_step, ++round) {
            const int rslot = f;
            gt_mbar_wait(red_full + rslot, round & 1, 4);
            // sum of the eight consumer warps, in warp order; lane l owns the values l + 32 j,
            // value i being (token i / 8, row i % 8) of the tile
            const float* red_u = red + rslot * GT_CWARPS * TILE_VALUES;
            float part[NW][GT_VPL];
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
                for (int j = 0; j < GT_VPL; ++j) {
                    float sum = 0.f;
#pragma unroll
                    for (int cw = 0; cw < GT_CWARPS; ++cw)
                        sum += red_u[cw * TILE_VALUES + w * (GT_ROWS * GT_TOK) + lane + 32 * j];
                    part[w][j] = sum;
                }
            __syncwarp();
            if (lane == 0) gt_mbar_arrive(red_empty + rslot);
            // The ranges of a tile meet in global memory without fences: a partial sum travels
            // as an 8-byte word (value, flag 1), which is written and read as one piece.  The
            // CTA of the last range collects: it polls the words of the ranges before it (CTAs
            // with smaller indices, which were scheduled before it), adds them in the order of
            // the ranges, its own last, and puts the words back to zero for the next launch.
            float2* tile_words = a.partials + (size_t)tile * (S - 1) * TILE_VALUES;
            if (split != S - 1) {
#pragma unroll
                for (int w = 0; w < NW; ++w)
#pragma unroll
                    for (int j = 0; j < GT_VPL; ++j)
                        __stcg(tile_words + split * TILE_VALUES + w * (GT_ROWS * GT_TOK) + lane + 32 * j,
                               make_float2(part[w][j], __int_as_float(1)));
                continue;
            }
            float total[NW][GT_VPL];
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
                for (int j = 0; j < GT_VPL; ++j) total[w][j] = 0.f;
            for (int sp = 0; sp < S - 1; ++sp) {
                float2* words = tile_words + sp * TILE_VALUES + lane;
                float value[NW][GT_VPL];
                gt_take_words<NW * GT_VPL>(words, &value[0][0]);
#pragma unroll
                for (int w = 0; w < NW; ++w)
#pragma unroll
                    for (int j = 0; j < GT_VPL; ++j) total[w][j] += value[w][j];
            }
#pragma unroll
            for (int j = 0; j < GT_VPL; ++j) {
                float v[NW];
#pragma unroll
                for (int w = 0; w < NW; ++w) v[w] = total[w][j] + part[w][j];
                const int idx = lane + 32 * j;
                const int tok = idx / GT_ROWS, feat = tile * GT_ROWS + (idx % GT_ROWS);
                const bool there = tok < a.M && feat < n_out;
                if (a.ss_in != nullptr) {
#pragma unroll
                    for (int w = 0; w < NW; ++w) v[w] *= inv_rms[tok];
                }
                if (!SWIGLU && a.resid != nullptr) {
                    // into the residual stream, and the next norm's input and share of squares
                    float r = 0.f;
                    if (there) {
                        r = a.resid[(int64_t)tok * a.ld_resid + feat] +
                            __bfloat162float(__float2bfloat16_rn(v[0]));
                        a.resid[(int64_t)tok * a.ld_resid + feat] = r;
                        a.x_out[(int64_t)tok * a.ld_xout + feat] = __float2bfloat16_rn(r * a.gain[feat]);
                    }
                    float sq = r * r;               // the 8 features of a token sit in 8 lanes
                    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                    if ((lane & 7) == 0) a.ss_out[(size_t)tile * GT_TOK + tok] = sq;
                } else if (there) {
                    float y = v[0];
                    if (SWIGLU) {
                        // the unfused path rounds gate and up to bfloat16 before the activation
                        const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
                        const float up = __bfloat162float(__float2bfloat16_rn(v[NW - 1]));
                        y = gate / (1.0f + expf(-gate)) * up;
                    }
                    gt_store(reinterpret_cast<TOut*>(a.Y) + (int64_t)tok * a.ldy + feat, y);
                }
            }
        }
        return;
    }

    // ---- consumers ----
    pdl_wait();
    pdl_trigger();
    // this CTA's slice of the activations: tokens beyond M are zero.  A thread requests eight
    // pieces before it stores the first, so that it waits for memory once per eight, not once
    // per piece.
    {
        const int chunks = n_st * GT_KS / 8;       // 16-byte pieces of a token row
        const int total = GT_TOK * chunks;
        constexpr int BATCH = 8, CT = GT_CWARPS * 32;
        for (int base = 0; base < total; base += BATCH * CT) {
            uint4 v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int idx = base + j * CT + tid;
                const int tok = idx / chunks, c = idx - tok * chunks;
                v[j] = make_uint4(0, 0, 0, 0);
                if (idx < total && tok < a.M)
                    v[j] = __ldcg(reinterpret_cast<const uint4*>(
                        a.X + (int64_t)tok * a.ldx + (int64_t)st_begin * GT_KS + c * 8));
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int idx = base + j * CT + tid;
                const int tok = idx / chunks, c = idx - tok * chunks;
                if (idx < total)
                    *reinterpret_cast<uint4*>(xs + (size_t)tok * a.x_stride + c * 8) = v[j];
            }
        }
    }
    gt_bar_sync(1, GT_CWARPS * 32);

    // Warp w takes the stages w, w + 8, ... of the CTA's sequence whole (the ring's depth is a
    // multiple of 8, so a slot always belongs to the same warp and the warp meets the phases of
    // the slot's barrier one after the other).  A barrier is then touched by one warp per stage,
    // and the warps work on eight stages at once.
    int it = 0, unit = 0;
    for (int tile = tile0; tile < tiles; tile += tile_step, ++unit) {
        float acc[NW][2][4];
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[w][h][e] = 0.f;
        for (int st = 0; st < n_st; ++st, ++it) {
            if ((it & (GT_CWARPS - 1)) != warp) continue;
            const int slot = it % stages;
            gt_mbar_wait(full + slot, (it / stages) & 1, 2);
            const unsigned char* stage = ring + (size_t)slot * STAGE_BYTES;
            // The tokens are the m of m16n8k16 (rows 8-15 of the A operand are zero and cost no
            // loads), 8 rows of W its n.  Element (row r, column k) of a block lies in the 64-column
            // chunk k / 64 at r * 128 + ((k % 64 / 8) ^ r) * 16: the 128-byte swizzle of the copy.
            const int r = lane & 7;
#pragma unroll
            for (int kk = 0; kk < GT_KS / 32; ++kk) {
                uint32_t xa[4];
                gt_ldsm_x4(xa, xs + (size_t)(lane & 7) * a.x_stride + st * GT_KS + kk * 32 +
                                   (lane >> 3) * 8);
                const int u = ((kk * 4 + (lane >> 3)) & 7) ^ r;   // 16-byte unit inside the 128-byte row
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    uint32_t wb[4];
                    gt_ldsm_x4(wb, stage + w * GT_BLOCK_BYTES + (kk >> 1) * (GT_ROWS * 128) + r * 128 +
                                       (u << 4));
                    gt_mma(acc[w][0], xa[0], xa[1], wb[0], wb[1]);
                    gt_mma(acc[w][1], xa[2], xa[3], wb[2], wb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) gt_mbar_arrive(empty + slot);
        }
        // hand the warp's partial sums to the combiner warps
        const int rslot = unit % F;
        if (unit >= F) gt_mbar_wait(red_empty + rslot, ((unit / F) - 1) & 1, 3);
        float* my_red = red + (rslot * GT_CWARPS + warp) * TILE_VALUES;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            // value tok * 8 + row of the tile; this lane holds token lane / 4, rows 2 (lane % 4), + 1
            float* dst = my_red + w * (GT_ROWS * GT_TOK) + (lane >> 2) * GT_ROWS + (lane & 3) * 2;
            dst[0] = acc[w][0][0] + acc[w][1][0];
            dst[1] = acc[w][0][1] + acc[w][1][1];
        }
        __syncwarp();
        if (lane == 0) gt_mbar_arrive(red_full + rslot);
    }
}

template <bool SWIGLU, typename TOut>
static int launch_gemv_tma(const CUtensorMap& map, const GemvTmaArgs& a, int grid, size_t smem,
                           cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_tma_kernel<SWIGLU, TOut>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM_LIMIT + 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return (int)sllm_launch_pdl(gemv_tma_kernel<SWIGLU, TOut>, dim3(grid), dim3(GT_THREADS), smem,
                                stream, map, a);
}

}  // namespace sllm

using namespace sllm;

// Ranges of K for a product.  One if the row tiles alone spread evenly over the CTAs (a very
// wide matrix); else two, or as many as keep a range within GT_MAX_RANGE.
static int gt_splits(int n_out, int K, int n_sm) {
    const int tiles = (n_out + GT_ROWS - 1) / GT_ROWS;
    // (measured at K = 4096: 12 row tiles per CTA are better off without the exchange between
    // ranges, 40.2 against 41.4 us; 3.5 are not, 8.7 against 8.2 us)
    if (tiles >= 8 * n_sm && (int64_t)GT_TOK * (K + 8) * 2 <= 72 * 1024) return 1;
    const int by_range = (K + GT_MAX_RANGE - 1) / GT_MAX_RANGE;
    return by_range > GT_MIN_SPLITS ? by_range : GT_MIN_SPLITS;
}
static int64_t gt_x_stride(int K, int S) {
    const int T = K / GT_KS;
    return (int64_t)((T + S - 1) / S) * GT_KS + 8;
}
// Barriers, hand-over slots and activations, rounded up so that the ring starts on 1024 bytes.
static int64_t gt_fixed_smem(int K, int S) {
    const int64_t bytes = 1024 + GT_RED_BYTES + GT_TOK * gt_x_stride(K, S) * 2;
    return (bytes + 1023) / 1024 * 1024;
}

typedef CUresult (*GtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// W [N, K] with row stride ldw as (64 columns, N rows, K / 64 chunks): one box is 16 rows of a
// stage's columns, stored chunk by chunk with the 128-byte swizzle.
static bool gt_make_map(CUtensorMap* map, const void* W, int N, int K, int64_t ldw) {
    static GtEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (GtEncodeTiledFn)p;
    }
    if (!fn) return false;
    cuuint64_t dims[3] = {64u, (cuuint64_t)N, (cuuint64_t)(K / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)ldw * 2, 128u};
    cuuint32_t box[3] = {64u, (cuuint32_t)GT_ROWS, (cuuint32_t)(GT_KS / 64)};
    cuuint32_t elem[3] = {1u, 1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(W), dims, strides, box,
              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Bytes of workspace a product needs: the words through which the ranges of K meet.
SLLM_EXPORT int64_t sllm_gemv_tma_workspace_bytes(int N, int K, int swiglu, int n_sm) {
    const int n_out = swiglu ? N / 2 : N;
    const int64_t tiles = (n_out + GT_ROWS - 1) / GT_ROWS;
    const int64_t values = (swiglu ? 2 : 1) * GT_ROWS * GT_TOK;
    return 16 + tiles * (gt_splits(n_out, K, n_sm) - 1) * values * 8;
}

// 1 if sllm_gemv_tma takes this product, 0 if another kernel has to.
SLLM_EXPORT int sllm_gemv_tma_supports(int M, int N, int K, int swiglu, int n_sm) {
    if (M < 1 || M > GT_TOK || N < 1 || (swiglu && (N % 2)) || n_sm < 1) return 0;
    const int S = gt_splits(swiglu ? N / 2 : N, K, n_sm);
    if (K % GT_KS || K / GT_KS < S || S > GT_MAX_SPLITS || S > n_sm) return 0;
    // the activations of a range, the hand-over slots and eight stages must fit
    const int nw = swiglu ? 2 : 1;
    return gt_fixed_smem(K, S) + GT_CWARPS * nw * GT_BLOCK_BYTES <= GT_SMEM_LIMIT ? 1 : 0;
}

// X [M, K], W [N, K] bfloat16 with rows 16-byte aligned; M <= 8.  swiglu = 0: Y [M, N];
// swiglu = 1: W = [gate rows; up rows], Y [M, N / 2].  out_dtype: 0 = float32, 1 = bfloat16.
// `workspace` holds sllm_gemv_tma_workspace_bytes(...) bytes that are zero before the first
// launch; launches leave them zero, so products of any sizes can share a workspace if their
// launches are ordered by their stream.  `n_sm`: SMs of the device.
// Deferred norm (see GemvTmaArgs): `ss_in` [ss_parts][8] with ss_dim and ss_eps makes the kernel
// multiply token t's outputs by rsqrt(sum_p ss_in[p][t] / ss_dim + ss_eps); `resid` (with
// ld_resid, gain [N], x_out with ld_xout, ss_out [ceil(N / 8)][8]; not with swiglu) makes it add
// its output into the residual stream and write the next norm's input and shares of squares
// instead of Y (which may then be nullptr).  nullptr switches either off.
SLLM_EXPORT int sllm_gemv_tma(const void* X, const void* W, void* Y, void* workspace, int M, int N,
                              int K, int64_t ldx, int64_t ldw, int64_t ldy, int swiglu,
                              int out_dtype, int n_sm, const float* ss_in, int ss_parts,
                              int ss_dim, float ss_eps, float* resid, int64_t ld_resid,
                              const float* gain, void* x_out, int64_t ld_xout, float* ss_out,
                              cudaStream_t stream) {
    if (!sllm_gemv_tma_supports(M, N, K, swiglu, n_sm)) return (int)cudaErrorInvalidValue;
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) ||
        ((uintptr_t)workspace & 15))
        return (int)cudaErrorInvalidValue;
    if (ss_in && (ss_parts < 1 || ss_dim < 1)) return (int)cudaErrorInvalidValue;
    if (resid && (swiglu || !gain || !x_out || !ss_out)) return (int)cudaErrorInvalidValue;
    if (!resid && !Y) return (int)cudaErrorInvalidValue;
    const int nw = swiglu ? 2 : 1;
    const int n_out = swiglu ? N / 2 : N;
    const int tiles = (n_out + GT_ROWS - 1) / GT_ROWS;
    const int S = gt_splits(n_out, K, n_sm);
    GemvTmaArgs a;
    a.X = (const bf16*)X;
    a.W = (const bf16*)W;
    a.Y = Y;
    a.partials = (float2*)workspace;
    a.M = M; a.N = N; a.K = K;
    a.ldx = ldx; a.ldw = ldw; a.ldy = ldy;
    a.splits = S;
    a.ss_in = ss_in; a.ss_parts = ss_parts;
    a.ss_inv_dim = ss_in ? 1.0f / (float)ss_dim : 0.f; a.ss_eps = ss_eps;
    a.resid = resid; a.ld_resid = ld_resid; a.gain = gain;
    a.x_out = (bf16*)x_out; a.ld_xout = ld_xout; a.ss_out = ss_out;
    a.x_stride = (int)gt_x_stride(K, S);
    const int64_t fixed = gt_fixed_smem(K, S);
    const int stage_bytes = nw * GT_BLOCK_BYTES;
    a.ring_offset = (int)fixed;
    CUtensorMap map;
    if (!gt_make_map(&map, W, N, K, ldw)) return (int)cudaErrorNotSupported;
    int stages = (int)((GT_SMEM_LIMIT - fixed) / stage_bytes);
    if (stages > GT_MAX_STAGES) stages = GT_MAX_STAGES;
    stages = stages / GT_CWARPS * GT_CWARPS;       // a slot always belongs to the same warp
    a.stages = stages;
    const size_t smem = (size_t)fixed + (size_t)stages * stage_bytes + 1024;
    int grid = (n_sm / S) * S;
    if (grid > tiles * S) grid = tiles * S;
    if (swiglu) {
        if (out_dtype == 1) return launch_gemv_tma<true, bf16>(map, a, grid, smem, stream);
        if (out_dtype == 0) return launch_gemv_tma<true, float>(map, a, grid, smem, stream);
    } else {
        if (out_dtype == 1) return launch_gemv_tma<false, bf16>(map, a, grid, smem, stream);
        if (out_dtype == 0) return launch_gemv_tma<false, float>(map, a, grid, smem, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// The first error recorded by a kernel since the last call (0 = none); clears it.
SLLM_EXPORT int sllm_gemv_tma_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_gemv_error, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_gemv_error, &zero, sizeof(int));
    return code;
}
