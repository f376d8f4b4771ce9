// Causal attention of a packed batch over the paged cache on the tensor cores (bfloat16
// operands, 32-bit accumulation and softmax): the serving path's attention for prefill
// portions and for decode.
//
// Restates src/scratch_llm/model.py:172-182 and :330-345 of the reference (scores scaled,
// disallowed keys -inf, softmax in 32-bit, probabilities rounded to the model dtype before
// they multiply v; query head h reads kv head h / (H/G)) as a tiled online-softmax kernel in
// the manner of its flash-attention oracle (src/scratch_llm/kernels/attention/reference.py:26-85).
// Like the reference's CUDA decode kernel (csrc/attention/a_r3_paged_decode_sm90.cu:32-39) a
// CTA serves one kv head and ALL query heads of its group, so keys and values are read once
// per group; unlike it, the products run on mma.sync tensor-core instructions, the head size
// and group size are free, and long rows are split over CTAs and merged by log-sum-exp
// (its merge: a_r3_paged_decode_sm90.cu:350-398).
//
// Work decomposition.  The queries of a row r and kv head g are "packed": packed index
// p = token * GS + j stands for the row's token `token` and query head g*GS + j (GS = H/G).
// A CTA takes BQ consecutive packed queries and walks the keys in tiles of 64 that are
// aligned to absolute positions.
//   wide  (SPLIT = false): BQ = 64; each of 4 warps owns 16 packed queries and all 64 keys
//                          of a tile.  For rows with many new tokens.
//   split (SPLIT = true):  BQ = 16; the 4 warps share the 16 packed queries and each takes
//                          16 keys of a tile; the key range is also split over `n_splits`
//                          CTAs whose partial results a merge kernel combines.  For decode.
//   column split (attn_decode_cs_kernel, head sizes that are multiples of 64): as split, but
//                          the probabilities of a tile meet in shared memory and each warp
//                          accumulates a quarter of the output columns over all 64 keys.
//                          The launcher uses it in place of split where it applies.
// Compiled once per head size: -DSLLM_HEAD_DIM=<multiple of 16, at most 256>.
#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#error "compile with -DSLLM_HEAD_DIM=<head size>"
#endif

namespace sllm {

constexpr int HD = SLLM_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size: a multiple of 16 up to 256");
constexpr int LDS = HD + 8;  // shared-memory row stride in elements: rows 16 bytes apart in banks
constexpr int BKV = 64, NWARP = 4, THREADS = 128;
constexpr int KSTEPS = HD / 16;  // k-steps of q k^T
constexpr int DTILES = HD / 8;   // 8-wide column tiles of the output
constexpr int CHUNKS = HD / 8;   // 16-byte chunks per row

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// d (16x8, f32) += a (16x16, bf16, row) * b (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <bool SPLIT> struct Mode {
    static constexpr int BQ = SPLIT ? 16 : 64;
    static constexpr int WKEYS = SPLIT ? BKV / NWARP : BKV;  // keys of a tile one warp takes
    static constexpr int NT = WKEYS / 8;                     // 8-wide score tiles per warp
    static constexpr int PK = WKEYS / 16;                    // k-steps of p v per warp
    // Pipeline depth.  Two stages leave room for three CTAs of the split kernel per SM; the
    // kernel is bound by instruction issue, so more resident warps pay more than deeper queues.
    static constexpr int NSTAGE = 2;
};

template <bool SPLIT> constexpr size_t smem_bytes() {
    return ((size_t)Mode<SPLIT>::BQ + 2 * Mode<SPLIT>::NSTAGE * BKV) * LDS * sizeof(bf16);
}

struct AttnArgs {
    const bf16* q; int64_t q_stride;
    const bf16* pages; const int* block_table; int table_stride; int page_size;
    const int* row_start; const int* row_pos0; const int* row_list;
    bf16* out; int64_t out_stride;
    float* part_o; float* part_lse; int n_splits;
    // tokens that part_o / part_lse have room for: a partial result of a token at or beyond
    // this index is not written (and *part_error is set, if given) instead of landing outside
    int64_t part_tokens; int* part_error;
    int H; int G; float scale_log2; int window;
    // attn_decode_cs_kernel only.  cos_t != nullptr: q, k and v are taken from the step's fused
    // projection as they are (q points at its first column): the kernel rotates q and the row's
    // new key itself and, if write_kv, stores the new key and value.
    const float* cos_t; const float* sin_t; int interleaved; int write_kv;
    // attn_decode_cs_kernel with several splits, one query tile per row: a counter per (listed
    // row, kv head), zero between launches.  The CTA that finishes last for a row and kv head
    // (it sees the count n_splits - 1) merges the splits' partial results itself, so that no
    // merge kernel follows; nobody waits for anybody.  nullptr: a merge kernel follows.
    int* merge_count;
};

template <bool SPLIT>
__global__ void __launch_bounds__(THREADS, SPLIT ? 3 : 2) attn_mma_kernel(const AttnArgs a) {
    using M = Mode<SPLIT>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + M::BQ * LDS;               // NSTAGE stages of [BKV][LDS]
    bf16* Vs = Ks + M::NSTAGE * BKV * LDS;     // NSTAGE stages of [BKV][LDS]

    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_splits = SPLIT ? a.n_splits : 1;
    // Query tiles in descending order: under the causal mask the last tile of a row has the
    // most keys to walk, and the longest jobs should start first.  CTAs start in the order of
    // blockIdx.x, then y, then z: the wide kernel (many tiles per row) therefore carries the
    // tile in z and the kv head in x, so that ALL heads' heaviest tiles start first; the split
    // kernel (one or a few tiles per row) keeps tiles and splits in x.
    const int q_tile = SPLIT ? (int)(gridDim.x / n_splits) - 1 - (int)(blockIdx.x / n_splits)
                             : (int)gridDim.z - 1 - (int)blockIdx.z;
    const int split = SPLIT ? blockIdx.x % n_splits : 0;
    const int r = a.row_list ? a.row_list[blockIdx.y] : blockIdx.y;
    const int g = SPLIT ? blockIdx.z : blockIdx.x;
    const int GS = a.H / a.G;
    const int t0 = a.row_start[r];
    const int n_new = a.row_start[r + 1] - t0;
    const int pos0 = a.row_pos0[r];
    const int n_packed = n_new * GS;
    const int q0 = q_tile * M::BQ;
    if (q0 >= n_packed) return;
    const int first_pos = pos0 + q0 / GS;
    const int last_pos = pos0 + min(n_packed - 1, q0 + M::BQ - 1) / GS;
    int k_lo = 0;
    if (a.window > 0) k_lo = max(0, first_pos - a.window + 1) / BKV * BKV;
    const int n_tiles = (last_pos - k_lo) / BKV + 1;
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int tile_begin = split * per_split;
    const int tile_end = min(n_tiles, tile_begin + per_split);

    // ---- queries into shared memory
    for (int idx = tid; idx < M::BQ * CHUNKS; idx += THREADS) {
        const int i = idx / CHUNKS, c = idx - i * CHUNKS;
        const int p = q0 + i;
        const bool valid = p < n_packed;
        const int tok = valid ? p / GS : 0, j = valid ? p - tok * GS : 0;
        const bf16* src = a.q + (int64_t)(t0 + tok) * a.q_stride + (int64_t)(g * GS + j) * HD + c * 8;
        cp_async16(Qs + i * LDS + c * 8, src, valid);
    }
    cp_async_commit();

    const int64_t v_off = (int64_t)a.G * a.page_size * HD;
    // Where a tile's keys live: thread j < 64 looks up key j's page once and leaves the element
    // offset of its K row in shared memory (-1: no such key); all threads then copy 16-byte
    // pieces from those offsets.  The lookup for a tile happens one step before its copy.
    __shared__ long long key_off[2][BKV];
    auto locate_tile = [&](int tile, int slot) {
        if (tid < BKV) {
            const int kpos = k_lo + tile * BKV + tid;
            long long off = -1;
            if (tile < tile_end && kpos <= last_pos) {
                const int page = a.block_table[(int64_t)r * a.table_stride + kpos / a.page_size];
                if (page >= 0)
                    off = (((long long)page * 2 * a.G + g) * a.page_size + kpos % a.page_size) * HD;
            }
            key_off[slot][tid] = off;
        }
    };
    constexpr int PIECES = BKV * CHUNKS / THREADS;
    static_assert(BKV * CHUNKS % THREADS == 0, "pieces per thread");
    auto load_tile = [&](int tile, int stage, int slot) {
        bf16* ks = Ks + stage * BKV * LDS;
        bf16* vs = Vs + stage * BKV * LDS;
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int idx = tid + i * THREADS;
            const int j = idx / CHUNKS, c = idx - j * CHUNKS;
            const long long off = key_off[slot][j];
            const bool ok = off >= 0;
            const bf16* src = ok ? a.pages + off + c * 8 : a.pages;
            cp_async16(ks + j * LDS + c * 8, src, ok);
            cp_async16(vs + j * LDS + c * 8, ok ? src + v_off : src, ok);
        }
    };

    // prologue: the first NSTAGE - 1 tiles (one commit group each, empty past the end)
    static_assert(M::NSTAGE == 2, "the key-offset slots below assume two stages");
    locate_tile(tile_begin, 0);
    __syncthreads();
    if (tile_begin < tile_end) load_tile(tile_begin, 0, 0);
    cp_async_commit();
    locate_tile(tile_begin + 1, 1);
    cp_async_wait<1>();  // the queries have landed (the first key tile may be in flight)
    __syncthreads();

    // ---- this warp's query fragments
    const int wq = SPLIT ? 0 : warp * 16;  // first packed query of the warp within the CTA
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
        ldsm_x4(qf[ks], Qs + (wq + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8);

    const int key_lo_w = SPLIT ? warp * M::WKEYS : 0;  // first key of a tile this warp takes
    // the two query rows of this thread: wq + lane/4 and wq + lane/4 + 8
    int qpos[2];
    bool qvalid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int p = q0 + wq + (lane >> 2) + 8 * h;
        qvalid[h] = p < n_packed;
        qpos[h] = pos0 + (qvalid[h] ? p / GS : 0);
    }
    // tiles that lie wholly before the warp's first query need no mask
    // (rows past the last packed query hold zeros, see the query load above: whatever they
    // compute stays finite and is never stored, so they do not force the masked path)
    const bool warp_full = a.window <= 0;
    const int warp_first_pos = pos0 + min(q0 + wq, n_packed - 1) / GS;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[DTILES][4];
#pragma unroll
    for (int dn = 0; dn < DTILES; ++dn)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dn][e] = 0.f;

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int stage = (tile - tile_begin) & 1;
        // offsets of tile + 1 were located one step ago (slot stage ^ 1) and are visible since
        // the barrier that ended that step
        if (tile + 1 < tile_end) load_tile(tile + 1, stage ^ 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();  // everything but the group just committed has landed
        __syncthreads();
        // slot `stage` was read by the copy issued one step ago; it is free for tile + 2
        locate_tile(tile + 2, stage);
        const bf16* ks_s = Ks + stage * BKV * LDS + key_lo_w * LDS;
        const bf16* vs_s = Vs + stage * BKV * LDS + key_lo_w * LDS;
        const int kt = k_lo + tile * BKV + key_lo_w;  // absolute position of the warp's key 0

        // ---- scores s = q k^T
        float s[M::NT][4];
#pragma unroll
        for (int nt = 0; nt < M::NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int nt = 0; nt < M::NT; nt += 2) {
                uint32_t b[4];
                ldsm_x4(b, ks_s + (nt * 8 + (lane & 7) + (lane >> 4) * 8) * LDS + ks * 16 +
                               ((lane >> 3) & 1) * 8);
                mma_bf16(s[nt], qf[ks], b[0], b[1]);
                mma_bf16(s[nt + 1], qf[ks], b[2], b[3]);
            }
        }
        // ---- mask, online softmax (base 2, in 32-bit)
        float mx[2] = {-INFINITY, -INFINITY};
        if (warp_full && kt + M::WKEYS - 1 <= warp_first_pos) {
#pragma unroll
            for (int nt = 0; nt < M::NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[nt][e] *= a.scale_log2;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < M::NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int kpos = kt + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const bool ok = qvalid[h] && kpos <= qpos[h] &&
                                    (a.window <= 0 || kpos > qpos[h] - a.window);
                    s[nt][e] = ok ? s[nt][e] * a.scale_log2 : -INFINITY;
                    mx[h] = fmaxf(mx[h], s[nt][e]);
                }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float m_new = fmaxf(m_run[h], quad_max(mx[h]));
            corr[h] = m_new == -INFINITY ? 1.f : exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
        uint32_t pa[M::PK][4];
#pragma unroll
        for (int nt = 0; nt < M::NT; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                p[e] = m_run[h] == -INFINITY ? 0.f : exp2f(s[nt][e] - m_run[h]);
                l_run[h] += p[e];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
        // the running maximum settles after the first tiles; skip the rescaling when no row
        // of the warp moved
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
            for (int dn = 0; dn < DTILES; ++dn) {
                o[dn][0] *= corr[0]; o[dn][1] *= corr[0];
                o[dn][2] *= corr[1]; o[dn][3] *= corr[1];
            }
        }
        // ---- o += p v
#pragma unroll
        for (int kk = 0; kk < M::PK; ++kk) {
#pragma unroll
            for (int dn = 0; dn < DTILES; dn += 2) {
                uint32_t b[4];
                ldsm_x4_trans(b, vs_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS +
                                     dn * 8 + (lane >> 4) * 8);
                mma_bf16(o[dn], pa[kk], b[0], b[1]);
                mma_bf16(o[dn + 1], pa[kk], b[2], b[3]);
            }
        }
        __syncthreads();  // this stage is overwritten by the load issued in the next iteration
    }
    cp_async_wait<0>();

    l_run[0] = quad_sum(l_run[0]);
    l_run[1] = quad_sum(l_run[1]);

    if (!SPLIT) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = q0 + wq + (lane >> 2) + 8 * h;
            if (p >= n_packed) continue;
            const int tok = p / GS, j = p - tok * GS;
            const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
            bf16* dst = a.out + (int64_t)(t0 + tok) * a.out_stride + (int64_t)(g * GS + j) * HD +
                        (lane & 3) * 2;
#pragma unroll
            for (int dn = 0; dn < DTILES; ++dn)
                *reinterpret_cast<__nv_bfloat162*>(dst + dn * 8) =
                    __floats2bfloat162_rn(o[dn][2 * h] * inv, o[dn][2 * h + 1] * inv);
        }
        return;
    }

    // ---- split mode: combine the four warps' partial results for the same 16 queries
    __syncthreads();  // all warps are done with the key and value stages
    float* sm_o = reinterpret_cast<float*>(Ks);           // [NWARP][16][HD]
    float* sm_m = sm_o + NWARP * 16 * HD;                  // [NWARP][16]
    float* sm_l = sm_m + NWARP * 16;                       // [NWARP][16]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int i = (lane >> 2) + 8 * h;
        if ((lane & 3) == 0) {
            sm_m[warp * 16 + i] = m_run[h];
            sm_l[warp * 16 + i] = l_run[h];
        }
#pragma unroll
        for (int dn = 0; dn < DTILES; ++dn) {
            float* dst = sm_o + ((warp * 16 + i) * HD) + dn * 8 + (lane & 3) * 2;
            dst[0] = o[dn][2 * h];
            dst[1] = o[dn][2 * h + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * HD; idx += THREADS) {
        const int i = idx / HD, d = idx - i * HD;
        const int p = q0 + i;
        if (p >= n_packed) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) mm = fmaxf(mm, sm_m[w * 16 + i]);
        float num = 0.f, den = 0.f;
        if (mm != -INFINITY) {
#pragma unroll
            for (int w = 0; w < NWARP; ++w) {
                const float f = exp2f(sm_m[w * 16 + i] - mm);
                num += f * sm_o[(w * 16 + i) * HD + d];
                den += f * sm_l[w * 16 + i];
            }
        }
        const float val = den > 0.f ? num / den : 0.f;
        const int tok = p / GS, j = p - tok * GS;
        const int64_t qh = (int64_t)(t0 + tok) * a.H + g * GS + j;  // (token, head) index
        if (n_splits == 1) {
            a.out[(int64_t)(t0 + tok) * a.out_stride + (int64_t)(g * GS + j) * HD + d] =
                __float2bfloat16_rn(val);
        } else if (t0 + tok < a.part_tokens) {
            a.part_o[(qh * n_splits + split) * HD + d] = val;
            if (d == 0)
                a.part_lse[qh * n_splits + split] = den > 0.f ? mm + log2f(den) : -INFINITY;
        } else if (a.part_error && d == 0) {
            *a.part_error = 1;   // the caller's token count does not cover this row
        }
    }
}

// Decode variant for head sizes that are multiples of 64.  Like the split kernel the four warps
// of a CTA share 16 packed queries and each computes the scores of 16 keys of a tile; but then
// the probabilities meet in shared memory and each warp accumulates ITS QUARTER OF THE OUTPUT
// COLUMNS over all 64 keys.  A warp therefore holds 16 x HD/4 of the output instead of 16 x HD
// (a quarter of the accumulator registers and of the rescaling work), the running maximum is
// common to the CTA, and no merge of four partial outputs is needed at the end.  The kernel
// is bound by instruction issue, and this is about a third of the split kernel's instructions.
#if SLLM_HEAD_DIM % 64 == 0
constexpr int CS_LDP = BKV + 8;        // row stride of the probability tile (elements)
constexpr int CS_OC = HD / NWARP;      // output columns per warp
constexpr int CS_OT = CS_OC / 8 > 0 ? CS_OC / 8 : 1;   // 8-wide output tiles per warp


__global__ void __launch_bounds__(THREADS, 3) attn_decode_cs_kernel(const AttnArgs a) {
    using M = Mode<true>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + M::BQ * LDS;
    bf16* Vs = Ks + M::NSTAGE * BKV * LDS;
    __shared__ long long key_off[2][BKV];
    // The probability tile takes the place of the queries once they are in registers (three
    // CTAs fit on an SM only if the static part stays small); the row sums reuse the maxima's.
    bf16* Ps = Qs;
    static_assert(CS_LDP <= LDS, "the probability tile must fit in the query tile");
    __shared__ float red_max[NWARP][16];
    float (*red_l)[16] = red_max;

    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_splits = a.n_splits;
    const int q_tile = (int)(gridDim.x / n_splits) - 1 - (int)(blockIdx.x / n_splits);
    const int split = blockIdx.x % n_splits;
    const int r = a.row_list ? a.row_list[blockIdx.y] : blockIdx.y;
    const int g = blockIdx.z;
    const int GS = a.H / a.G;
    const int t0 = a.row_start[r];
    const int n_new = a.row_start[r + 1] - t0;
    const int pos0 = a.row_pos0[r];
    const int n_packed = n_new * GS;
    const int q0 = q_tile * M::BQ;
    if (q0 >= n_packed) return;
    const int first_pos = pos0 + q0 / GS;
    const int last_pos = pos0 + min(n_packed - 1, q0 + M::BQ - 1) / GS;
    int k_lo = 0;
    if (a.window > 0) k_lo = max(0, first_pos - a.window + 1) / BKV * BKV;
    const int n_tiles = (last_pos - k_lo) / BKV + 1;
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int tile_begin = split * per_split;
    const int tile_end = min(n_tiles, tile_begin + per_split);

    for (int idx = tid; idx < M::BQ * CHUNKS; idx += THREADS) {
        const int i = idx / CHUNKS, c = idx - i * CHUNKS;
        const int p = q0 + i;
        const bool valid = p < n_packed;
        const int tok = valid ? p / GS : 0, j = valid ? p - tok * GS : 0;
        const bf16* src = a.q + (int64_t)(t0 + tok) * a.q_stride + (int64_t)(g * GS + j) * HD + c * 8;
        cp_async16(Qs + i * LDS + c * 8, src, valid);
    }
    cp_async_commit();

    const int64_t v_off = (int64_t)a.G * a.page_size * HD;
    // With the rotation fused (rows of one new token at position pos0): everything it needs
    // from global memory is requested now, so that it has arrived when the tiles have.
    // Thread t rotates pair t % (HD / 2) of the query heads t / (HD / 2), ... and of the new key,
    // and carries element t, t + THREADS, ... of the new value.
    const bool fused_rope = a.cos_t != nullptr;
    const int new_tile = fused_rope && a.write_kv ? (pos0 - k_lo) / BKV : -1;
    const bool owns_new = new_tile >= tile_begin && new_tile < tile_end;
    constexpr int HALF = HD / 2;
    constexpr int V_PER = (HD + THREADS - 1) / THREADS, K_PER = (HALF + THREADS - 1) / THREADS;
    float rope_c[K_PER], rope_s[K_PER];
    __nv_bfloat162 k_new[K_PER];
    bf16 v_new[V_PER];
    if (fused_rope) {
#pragma unroll
        for (int u = 0; u < K_PER; ++u) {
            const int j = tid + u * THREADS;
            if (j < HALF) {
                rope_c[u] = a.cos_t[(int64_t)pos0 * HALF + j];
                rope_s[u] = a.sin_t[(int64_t)pos0 * HALF + j];
            }
        }
        if (owns_new) {
            const bf16* k_src = a.q + (int64_t)t0 * a.q_stride + (int64_t)(a.H + g) * HD;
            const bf16* v_src = k_src + (int64_t)a.G * HD;
#pragma unroll
            for (int u = 0; u < K_PER; ++u) {
                const int j = tid + u * THREADS;
                if (j < HALF) {
                    const int i0 = a.interleaved ? 2 * j : j, i1 = a.interleaved ? 2 * j + 1 : j + HALF;
                    k_new[u] = __halves2bfloat162(k_src[i0], k_src[i1]);
                }
            }
#pragma unroll
            for (int u = 0; u < V_PER; ++u)
                if (tid + u * THREADS < HD) v_new[u] = v_src[tid + u * THREADS];
        }
    }
    auto locate_tile = [&](int tile, int slot) {
        if (tid < BKV) {
            const int kpos = k_lo + tile * BKV + tid;
            long long off = -1;
            if (tile < tile_end && kpos <= last_pos) {
                const int page = a.block_table[(int64_t)r * a.table_stride + kpos / a.page_size];
                if (page >= 0)
                    off = (((long long)page * 2 * a.G + g) * a.page_size + kpos % a.page_size) * HD;
            }
            key_off[slot][tid] = off;
        }
    };
    constexpr int PIECES = BKV * CHUNKS / THREADS;
    auto load_tile = [&](int tile, int stage, int slot) {
        bf16* ks = Ks + stage * BKV * LDS;
        bf16* vs = Vs + stage * BKV * LDS;
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int idx = tid + i * THREADS;
            const int j = idx / CHUNKS, c = idx - j * CHUNKS;
            const long long off = key_off[slot][j];
            const bool ok = off >= 0;
            const bf16* src = ok ? a.pages + off + c * 8 : a.pages;
            cp_async16(ks + j * LDS + c * 8, src, ok);
            cp_async16(vs + j * LDS + c * 8, ok ? src + v_off : src, ok);
        }
    };
    locate_tile(tile_begin, 0);
    __syncthreads();
    if (tile_begin < tile_end) load_tile(tile_begin, 0, 0);
    cp_async_commit();
    locate_tile(tile_begin + 1, 1);
    cp_async_wait<1>();
    __syncthreads();
    if (fused_rope) {
        // q as the projection left it: rotate the row's GS heads here (32-bit, one rounding,
        // the arithmetic of rope_cache.cu)
#pragma unroll
        for (int u = 0; u < K_PER; ++u) {
            const int j = tid + u * THREADS;
            if (j < HALF) {
                const int i0 = a.interleaved ? 2 * j : j, i1 = a.interleaved ? 2 * j + 1 : j + HALF;
                for (int i = 0; i < GS; ++i) {
                    const float x0 = __bfloat162float(Qs[i * LDS + i0]);
                    const float x1 = __bfloat162float(Qs[i * LDS + i1]);
                    Qs[i * LDS + i0] = __float2bfloat16_rn(x0 * rope_c[u] - x1 * rope_s[u]);
                    Qs[i * LDS + i1] = __float2bfloat16_rn(x0 * rope_s[u] + x1 * rope_c[u]);
                }
            }
        }
        __syncthreads();
    }

    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
        ldsm_x4(qf[ks], Qs + (lane & 15) * LDS + ks * 16 + (lane >> 4) * 8);
    const int key_lo_w = warp * M::WKEYS;
    int qpos[2];
    bool qvalid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int p = q0 + (lane >> 2) + 8 * h;
        qvalid[h] = p < n_packed;
        qpos[h] = pos0 + (qvalid[h] ? p / GS : 0);
    }
    const bool no_window = a.window <= 0;
    const int first_q_pos = pos0 + min(q0, n_packed - 1) / GS;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[CS_OT][4];
#pragma unroll
    for (int dn = 0; dn < CS_OT; ++dn)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dn][e] = 0.f;

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int stage = (tile - tile_begin) & 1;
        if (tile + 1 < tile_end) load_tile(tile + 1, stage ^ 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        locate_tile(tile + 2, stage);
        if (tile == new_tile) {
            // the row's new key (rotated here) and value: into the cache for the steps to come,
            // and over what the copy fetched from that place of the cache for this one
            const int in_tile = pos0 - k_lo - tile * BKV;
            bf16* k_row = Ks + stage * BKV * LDS + in_tile * LDS;
            bf16* v_row = Vs + stage * BKV * LDS + in_tile * LDS;
            const int page = a.block_table[(int64_t)r * a.table_stride + pos0 / a.page_size];
            bf16* k_dst = const_cast<bf16*>(a.pages) +
                          (((long long)page * 2 * a.G + g) * a.page_size + pos0 % a.page_size) * HD;
            bf16* v_dst = k_dst + v_off;
#pragma unroll
            for (int u = 0; u < K_PER; ++u) {
                const int j = tid + u * THREADS;
                if (j < HALF) {
                    const int i0 = a.interleaved ? 2 * j : j, i1 = a.interleaved ? 2 * j + 1 : j + HALF;
                    const float x0 = __low2float(k_new[u]), x1 = __high2float(k_new[u]);
                    const bf16 r0 = __float2bfloat16_rn(x0 * rope_c[u] - x1 * rope_s[u]);
                    const bf16 r1 = __float2bfloat16_rn(x0 * rope_s[u] + x1 * rope_c[u]);
                    k_row[i0] = r0; k_row[i1] = r1;
                    k_dst[i0] = r0; k_dst[i1] = r1;
                }
            }
#pragma unroll
            for (int u = 0; u < V_PER; ++u) {
                const int i = tid + u * THREADS;
                if (i < HD) {
                    v_row[i] = v_new[u];
                    v_dst[i] = v_new[u];
                }
            }
            __syncthreads();
        }
        const bf16* ks_s = Ks + stage * BKV * LDS + key_lo_w * LDS;
        const bf16* vs_s = Vs + stage * BKV * LDS;
        const int kt = k_lo + tile * BKV + key_lo_w;

        // scores of this warp's 16 keys
        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t b[4];
            ldsm_x4(b, ks_s + ((lane & 7) + (lane >> 4) * 8) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[0], qf[ks], b[0], b[1]);
            mma_bf16(s[1], qf[ks], b[2], b[3]);
        }
        float mx[2] = {-INFINITY, -INFINITY};
        if (no_window && kt + M::WKEYS - 1 <= first_q_pos) {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[nt][e] *= a.scale_log2;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int kpos = kt + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const bool ok = qvalid[h] && kpos <= qpos[h] &&
                                    (a.window <= 0 || kpos > qpos[h] - a.window);
                    s[nt][e] = ok ? s[nt][e] * a.scale_log2 : -INFINITY;
                    mx[h] = fmaxf(mx[h], s[nt][e]);
                }
        }
        mx[0] = quad_max(mx[0]);
        mx[1] = quad_max(mx[1]);
        if ((lane & 3) == 0) {
            red_max[warp][lane >> 2] = mx[0];
            red_max[warp][(lane >> 2) + 8] = mx[1];
        }
        __syncthreads();   // the four warps' maxima of this tile are in place
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const float mt = fmaxf(fmaxf(red_max[0][row], red_max[1][row]),
                                   fmaxf(red_max[2][row], red_max[3][row]));
            const float m_new = fmaxf(m_run[h], mt);
            corr[h] = m_new == -INFINITY ? 1.f : exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                p[e] = m_run[h] == -INFINITY ? 0.f : exp2f(s[nt][e] - m_run[h]);
                l_run[h] += p[e];
            }
            bf16* dst = Ps + (lane >> 2) * CS_LDP + key_lo_w + nt * 8 + (lane & 3) * 2;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(p[0], p[1]);
            *reinterpret_cast<__nv_bfloat162*>(dst + 8 * CS_LDP) = __floats2bfloat162_rn(p[2], p[3]);
        }
        if (corr[0] != 1.f || corr[1] != 1.f) {   // same in every thread of a row's quad
#pragma unroll
            for (int dn = 0; dn < CS_OT; ++dn) {
                o[dn][0] *= corr[0]; o[dn][1] *= corr[0];
                o[dn][2] *= corr[1]; o[dn][3] *= corr[1];
            }
        }
        __syncthreads();   // the probabilities of all 64 keys are in place
        // this warp's columns of the output over all 64 keys
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            uint32_t pa[4];
            ldsm_x4(pa, Ps + (lane & 15) * CS_LDP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int dn = 0; dn < CS_OT; dn += 2) {
                uint32_t b[4];
                ldsm_x4_trans(b, vs_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS +
                                     warp * CS_OC + dn * 8 + (lane >> 4) * 8);
                mma_bf16(o[dn], pa, b[0], b[1]);
                mma_bf16(o[dn + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();   // stage, probabilities and maxima are reused by the next tile
    }
    cp_async_wait<0>();

    // the sum of the probabilities over the four warps' keys
    l_run[0] = quad_sum(l_run[0]);
    l_run[1] = quad_sum(l_run[1]);
    if ((lane & 3) == 0) {
        red_l[warp][lane >> 2] = l_run[0];
        red_l[warp][(lane >> 2) + 8] = l_run[1];
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = (lane >> 2) + 8 * h;
        const int p = q0 + row;
        if (p >= n_packed) continue;
        const float l_tot = (red_l[0][row] + red_l[1][row]) + (red_l[2][row] + red_l[3][row]);
        const float inv = l_tot > 0.f ? 1.0f / l_tot : 0.f;
        const int tok = p / GS, j = p - tok * GS;
        const int col0 = warp * CS_OC + (lane & 3) * 2;
        if (n_splits == 1) {
            bf16* dst = a.out + (int64_t)(t0 + tok) * a.out_stride + (int64_t)(g * GS + j) * HD + col0;
#pragma unroll
            for (int dn = 0; dn < CS_OT; ++dn)
                *reinterpret_cast<__nv_bfloat162*>(dst + dn * 8) =
                    __floats2bfloat162_rn(o[dn][2 * h] * inv, o[dn][2 * h + 1] * inv);
        } else if (t0 + tok >= a.part_tokens) {
            if (a.part_error && warp == 0 && (lane & 3) == 0) *a.part_error = 1;
        } else {
            const int64_t qh = (int64_t)(t0 + tok) * a.H + g * GS + j;
            float* dst = a.part_o + (qh * n_splits + split) * HD + col0;
#pragma unroll
            for (int dn = 0; dn < CS_OT; ++dn) {
                dst[dn * 8] = o[dn][2 * h] * inv;
                dst[dn * 8 + 1] = o[dn][2 * h + 1] * inv;
            }
            if (warp == 0 && (lane & 3) == 0)
                a.part_lse[qh * n_splits + split] =
                    l_tot > 0.f ? m_run[h] + log2f(l_tot) : -INFINITY;
        }
    }
    if (n_splits > 1 && a.merge_count != nullptr) {
        // The last CTA to arrive for this row and kv head merges (the arithmetic and the order
        // of attn_merge_kernel: the result does not depend on which CTA that is).  The fence
        // before the count makes this CTA's partial results visible to whoever counts later.
        __shared__ int is_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int* count = a.merge_count + (size_t)blockIdx.y * a.G + g;
            is_last = atomicAdd(count, 1) == n_splits - 1;
            if (is_last) *count = 0;                 // zero again for the next launch
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        for (int idx = tid; idx < n_packed * (HD / 4); idx += THREADS) {
            const int p = idx / (HD / 4), d = (idx - p * (HD / 4)) * 4;
            const int tok = p / GS, j = p - tok * GS;
            if (t0 + tok >= a.part_tokens) continue;
            const int64_t qh = (int64_t)(t0 + tok) * a.H + g * GS + j;
            const float* lse = a.part_lse + qh * n_splits;
            float mm = -INFINITY;
            for (int sp = 0; sp < n_splits; ++sp) mm = fmaxf(mm, __ldcg(lse + sp));
            float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.f;
            if (mm != -INFINITY) {
                const float* po = a.part_o + qh * n_splits * HD + d;
#pragma unroll 8
                for (int sp = 0; sp < n_splits; ++sp) {
                    const float f = exp2f(__ldcg(lse + sp) - mm);
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(po + (int64_t)sp * HD));
                    num.x += f * v.x;
                    num.y += f * v.y;
                    num.z += f * v.z;
                    num.w += f * v.w;
                    den += f;
                }
            }
            const bool some = den > 0.f;
            bf16* dst = a.out + (int64_t)(t0 + tok) * a.out_stride + (int64_t)(g * GS + j) * HD + d;
            *reinterpret_cast<__nv_bfloat162*>(dst) =
                __floats2bfloat162_rn(some ? num.x / den : 0.f, some ? num.y / den : 0.f);
            *reinterpret_cast<__nv_bfloat162*>(dst + 2) =
                __floats2bfloat162_rn(some ? num.z / den : 0.f, some ? num.w / den : 0.f);
        }
    }
}

#endif  // SLLM_HEAD_DIM % 64 == 0

// Combines the partial results of the splits: o = sum_s 2^(lse_s - m) o_s / sum_s 2^(lse_s - m).
// grid (listed rows, H / 4), 4 warps: a warp takes one head and walks the row's tokens; a lane
// takes 4 consecutive elements of the head at a time.  The sums run over the splits in their
// order (so the result does not depend on the launch's shape); the loop is unrolled so that
// the loads of several splits are in flight at once.
constexpr int MERGE_WARPS = 4;
__global__ void __launch_bounds__(MERGE_WARPS * 32) attn_merge_kernel(
        const float* __restrict__ part_o, const float* __restrict__ part_lse, int n_splits,
        const int* __restrict__ row_start, const int* __restrict__ row_list,
        bf16* __restrict__ out, int64_t out_stride, int H, int64_t part_tokens) {
    pdl_wait();
    pdl_trigger();
    const int r = row_list ? row_list[blockIdx.x] : blockIdx.x;
    const int head = blockIdx.y * MERGE_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= H) return;
    // (tokens beyond what the partial arrays cover were not written: they are left out here too)
    const int t_end = (int)min((int64_t)row_start[r + 1], part_tokens);
    for (int t = row_start[r]; t < t_end; ++t) {
        const int64_t qh = (int64_t)t * H + head;
        const float* lse = part_lse + qh * n_splits;
        float mm = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) mm = fmaxf(mm, lse[s]);
        mm = warp_max(mm);
        for (int d = lane * 4; d < HD; d += 128) {
            float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.f;
            if (mm != -INFINITY) {
                const float* o = part_o + qh * n_splits * HD + d;
#pragma unroll 8
                for (int s = 0; s < n_splits; ++s) {
                    const float f = exp2f(lse[s] - mm);
                    const float4 v = *reinterpret_cast<const float4*>(o + (int64_t)s * HD);
                    num.x += f * v.x;
                    num.y += f * v.y;
                    num.z += f * v.z;
                    num.w += f * v.w;
                    den += f;
                }
            }
            const bool some = den > 0.f;
            __nv_bfloat162 lo = __floats2bfloat162_rn(some ? num.x / den : 0.f, some ? num.y / den : 0.f);
            __nv_bfloat162 hi = __floats2bfloat162_rn(some ? num.z / den : 0.f, some ? num.w / den : 0.f);
            bf16* dst = out + (int64_t)t * out_stride + (int64_t)head * HD + d;
            // out_stride is even and HD a multiple of 16: 4-byte stores are aligned
            *reinterpret_cast<__nv_bfloat162*>(dst) = lo;
            *reinterpret_cast<__nv_bfloat162*>(dst + 2) = hi;
        }
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attn_mma_head_dim() { return HD; }

// CTAs of the split (decode) kernel that the current device holds at once: SMs x the CTAs of
// that kernel resident on one SM (from the occupancy calculator).  0 on an error.
SLLM_EXPORT int sllm_attn_mma_decode_slots() {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    const size_t smem = smem_bytes<true>();
#if SLLM_HEAD_DIM % 64 == 0
    if (cudaFuncSetAttribute(attn_decode_cs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_cs_kernel, THREADS,
                                                      smem) != cudaSuccess) return 0;
#else
    if (cudaFuncSetAttribute(attn_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_mma_kernel<true>, THREADS,
                                                      smem) != cudaSuccess) return 0;
#endif
    return sms * per_sm;
}

// Scratch floats the split kernel needs for `n_tokens` tokens in its listed rows.
SLLM_EXPORT int64_t sllm_attn_mma_scratch_floats(int64_t n_tokens, int H, int n_splits) {
    return n_splits > 1 ? n_tokens * H * n_splits * (HD + 1) : 0;
}

// q / out: [n_tokens, stride] bfloat16 with head h at columns [h*HD, (h+1)*HD).
// pages: [n_pages, 2, G, page_size, HD] bfloat16.  block_table: [rows, table_stride], -1 = none.
// row_list: the n_list rows this launch serves (nullptr: rows 0..n_list-1).
// split = 0: the wide kernel; max_new = the largest number of new tokens of a listed row.
// split = 1: the split kernel with n_splits CTAs along the keys; for n_splits > 1,
//            `scratch` holds sllm_attn_mma_scratch_floats(total tokens of the batch, H, n_splits)
//            floats and a merge kernel writes the result.
SLLM_EXPORT int sllm_attn_mma(const void* q, int64_t q_stride, const void* pages,
                              const int* block_table, int table_stride, int page_size,
                              const int* row_start, const int* row_pos0, const int* row_list,
                              int n_list, int max_new, void* out, int64_t out_stride, int H, int G,
                              float scale, int window, int split, int n_splits, float* scratch,
                              int64_t n_tokens_total, cudaStream_t stream) {
    if (n_list <= 0 || max_new <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || page_size <= 0 || window < 0 || n_list > 65535 ||
        G > 65535 || (q_stride % 8) != 0 || (out_stride % 2) != 0)
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)q & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3))
        return (int)cudaErrorInvalidValue;
    AttnArgs a;
    a.q = (const bf16*)q; a.q_stride = q_stride;
    a.pages = (const bf16*)pages; a.block_table = block_table; a.table_stride = table_stride;
    a.page_size = page_size; a.row_start = row_start; a.row_pos0 = row_pos0; a.row_list = row_list;
    a.out = (bf16*)out; a.out_stride = out_stride;
    a.part_o = nullptr; a.part_lse = nullptr; a.n_splits = 1;
    a.part_tokens = n_tokens_total; a.part_error = nullptr; a.merge_count = nullptr;
    a.cos_t = nullptr; a.sin_t = nullptr; a.interleaved = 1; a.write_kv = 0;
    a.H = H; a.G = G; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
    const int GS = H / G;
    cudaError_t e;
    if (!split) {
        const size_t smem = smem_bytes<false>();
        e = cudaFuncSetAttribute(attn_mma_kernel<false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        const int64_t q_tiles = ((int64_t)max_new * GS + 63) / 64;
        if (q_tiles > 65535) return (int)cudaErrorInvalidValue;   // the tiles are the grid's z
        dim3 grid(G, n_list, (unsigned)q_tiles);
        return (int)sllm_launch_pdl(attn_mma_kernel<false>, grid, dim3(THREADS), smem, stream, a);
    }
    if (n_splits < 1) return (int)cudaErrorInvalidValue;
    if (n_splits > 1) {
        if (!scratch) return (int)cudaErrorInvalidValue;
        a.part_o = scratch;
        a.part_lse = scratch + n_tokens_total * H * n_splits * HD;
    }
    a.n_splits = n_splits;
    const size_t smem = smem_bytes<true>();
    e = cudaFuncSetAttribute(attn_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((((int64_t)max_new * GS + 15) / 16) * n_splits, n_list, G);
#if SLLM_HEAD_DIM % 64 == 0
    e = cudaFuncSetAttribute(attn_decode_cs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = sllm_launch_pdl(attn_decode_cs_kernel, grid, dim3(THREADS), smem, stream, a);
#else
    e = sllm_launch_pdl(attn_mma_kernel<true>, grid, dim3(THREADS), smem, stream, a);
#endif
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        dim3 mgrid(n_list, (H + MERGE_WARPS - 1) / MERGE_WARPS);
        e = sllm_launch_pdl(attn_merge_kernel, mgrid, dim3(MERGE_WARPS * 32), 0, stream,
                            (const float*)a.part_o, (const float*)a.part_lse, n_splits, row_start,
                            row_list, (bf16*)out, out_stride, H, a.part_tokens);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

#if SLLM_HEAD_DIM % 64 == 0
// 1: this head size has the decode kernel that can rotate q and the new key and store the new
// key and value itself.
SLLM_EXPORT int sllm_attn_mma_decode_fused_supported() { return 1; }

// The decode kernel for rows of ONE new token (groups of up to 16 query heads) that takes q, k
// and v as the projection left them.  cos_t / sin_t: [positions, HD / 2] float tables; `qkv` is
// the step's fused projection [tokens, (H + 2 G) * HD] (q heads, k heads, v heads); the kernel
// rotates q and the new key (adjacent pairs if `interleaved`, else the halves) and, if
// `write_kv`, stores the rotated key and the value at the row's position in the cache.
// `scratch` as in sllm_attn_mma for n_splits > 1.  `merge_count`: n_list * G counters that are
// zero before the first launch (every launch leaves them zero): the CTA that finishes last for
// a row and kv head merges the splits itself; nullptr: a merge kernel follows instead.
SLLM_EXPORT int sllm_attn_mma_decode(const void* qkv, int64_t qkv_stride, void* pages,
                                     const int* block_table, int table_stride, int page_size,
                                     const int* row_start, const int* row_pos0,
                                     const int* row_list, int n_list, void* out,
                                     int64_t out_stride, int H, int G, float scale, int window,
                                     int n_splits, float* scratch, int64_t n_tokens_total,
                                     const float* cos_t, const float* sin_t, int interleaved,
                                     int write_kv, int* merge_count, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || page_size <= 0 || window < 0 || n_list > 65535 ||
        G > 65535 || (qkv_stride % 8) != 0 || (out_stride % 2) != 0 || n_splits < 1 || H / G > 16)
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)qkv & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3) || !cos_t || !sin_t)
        return (int)cudaErrorInvalidValue;
    AttnArgs a;
    a.q = (const bf16*)qkv; a.q_stride = qkv_stride;
    a.pages = (const bf16*)pages; a.block_table = block_table; a.table_stride = table_stride;
    a.page_size = page_size; a.row_start = row_start; a.row_pos0 = row_pos0; a.row_list = row_list;
    a.out = (bf16*)out; a.out_stride = out_stride;
    a.part_o = nullptr; a.part_lse = nullptr; a.n_splits = n_splits;
    a.part_tokens = n_tokens_total; a.part_error = nullptr;
    a.merge_count = n_splits > 1 ? merge_count : nullptr;
    a.H = H; a.G = G; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
    a.cos_t = cos_t; a.sin_t = sin_t; a.interleaved = interleaved; a.write_kv = write_kv;
    if (n_splits > 1) {
        if (!scratch) return (int)cudaErrorInvalidValue;
        a.part_o = scratch;
        a.part_lse = scratch + n_tokens_total * H * n_splits * HD;
    }
    const size_t smem = smem_bytes<true>();
    cudaError_t e = cudaFuncSetAttribute(attn_decode_cs_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(n_splits, n_list, G);   // one tile of 16 packed queries per (row, kv head)
    e = sllm_launch_pdl(attn_decode_cs_kernel, grid, dim3(THREADS), smem, stream, a);
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1 && a.merge_count == nullptr) {
        dim3 mgrid(n_list, (H + MERGE_WARPS - 1) / MERGE_WARPS);
        e = sllm_launch_pdl(attn_merge_kernel, mgrid, dim3(MERGE_WARPS * 32), 0, stream,
                            (const float*)a.part_o, (const float*)a.part_lse, n_splits, row_start,
                            row_list, (bf16*)out, out_stride, H, a.part_tokens);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}
#else
SLLM_EXPORT int sllm_attn_mma_decode_fused_supported() { return 0; }
#endif

// ------------------------------------------------------------------------------------------
// The split kernel for callers that must not allocate: see attention_mma_noalloc.h.
#include <stdio.h>

#include "attention_mma_noalloc.h"

// Scratch for the partial results.  In host code this name is only a handle for
// cudaGetSymbolAddress: it is not a device address and must never be passed to a kernel.
static __device__ __align__(256) float g_noalloc_scratch[SLLM_NOALLOC_SCRATCH_FLOATS];
// Set by a kernel that met a token at or beyond n_tokens_total (its partial result was left out
// instead of being written outside the array).
static __device__ int g_noalloc_overrun;

static float* g_noalloc_ptr[64];     // device address of the array, per device ordinal
static int* g_noalloc_flag_ptr[64];  // device address of the overrun flag, per device ordinal
static char g_noalloc_error[256] = "";

SLLM_EXPORT int64_t sllm_attn_mma_noalloc_capacity_floats(void) {
    return SLLM_NOALLOC_SCRATCH_FLOATS;
}

SLLM_EXPORT const char* sllm_attn_mma_noalloc_error(void) { return g_noalloc_error; }

SLLM_EXPORT int sllm_attn_mma_noalloc_overrun(void) {
    int flag = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&flag, g_noalloc_overrun, sizeof(int)) != cudaSuccess) return -1;
    if (flag && cudaMemcpyToSymbol(g_noalloc_overrun, &zero, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}

SLLM_EXPORT int sllm_attn_mma_split_noalloc(const void* q, int64_t q_stride, const void* pages,
                                            const int* block_table, int table_stride,
                                            int page_size, const int* row_start,
                                            const int* row_pos0, const int* row_list, int n_list,
                                            int max_new, void* out, int64_t out_stride, int H,
                                            int G, float scale, int window, int n_splits,
                                            int64_t n_tokens_total, cudaStream_t stream) {
    if (n_list <= 0 || max_new <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || page_size <= 0 || window < 0 || n_list > 65535 ||
        G > 65535 || H > 65535 || (q_stride % 8) != 0 || (out_stride % 2) != 0 || n_splits < 1 ||
        n_splits > SLLM_NOALLOC_MAX_SPLITS || n_tokens_total < 0 ||
        n_tokens_total > (int64_t)SLLM_NOALLOC_SCRATCH_FLOATS) {
        // (the bounds on H, n_splits and n_tokens_total also keep the product below from
        // overflowing 64 bits)
        snprintf(g_noalloc_error, sizeof(g_noalloc_error),
                 "sllm_attn_mma_split_noalloc: an argument is out of range (1 <= n_splits <= %d, "
                 "0 <= n_tokens_total <= %lld, strides of q a multiple of 8 and of out even)",
                 SLLM_NOALLOC_MAX_SPLITS, (long long)SLLM_NOALLOC_SCRATCH_FLOATS);
        return (int)cudaErrorInvalidValue;
    }
    if (((uintptr_t)q & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3))
        return (int)cudaErrorInvalidValue;
    const int64_t need = sllm_attn_mma_scratch_floats(n_tokens_total, H, n_splits);
    if (need > (int64_t)SLLM_NOALLOC_SCRATCH_FLOATS) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error),
                 "sllm_attn_mma_split_noalloc: %lld tokens x %d heads x %d splits need %lld "
                 "scratch floats, the built-in array holds %lld: use fewer splits or tokens, or "
                 "sllm_attn_mma with scratch of your own",
                 (long long)n_tokens_total, H, n_splits, (long long)need,
                 (long long)SLLM_NOALLOC_SCRATCH_FLOATS);
        return (int)cudaErrorInvalidValue;
    }
    // set-up, once per device, with that device current
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (g_noalloc_ptr[dev] == nullptr) {
        float* ptr = nullptr;
        int* flag = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        e = cudaGetSymbolAddress((void**)&flag, g_noalloc_overrun);
        if (e != cudaSuccess) return (int)e;
        g_noalloc_flag_ptr[dev] = flag;
        g_noalloc_ptr[dev] = ptr;
    }
    float* scratch = g_noalloc_ptr[dev];

    AttnArgs a{};   // (the fields of the fused decode kernel stay null / 0: it is not used here)
    a.q = (const bf16*)q; a.q_stride = q_stride;
    a.pages = (const bf16*)pages; a.block_table = block_table; a.table_stride = table_stride;
    a.page_size = page_size; a.row_start = row_start; a.row_pos0 = row_pos0; a.row_list = row_list;
    a.out = (bf16*)out; a.out_stride = out_stride;
    a.part_o = n_splits > 1 ? scratch : nullptr;
    a.part_lse = n_splits > 1 ? scratch + n_tokens_total * H * n_splits * HD : nullptr;
    a.n_splits = n_splits;
    a.part_tokens = n_tokens_total; a.part_error = g_noalloc_flag_ptr[dev];
    a.cos_t = nullptr; a.sin_t = nullptr; a.interleaved = 1; a.write_kv = 0;
    a.H = H; a.G = G; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
    const int GS = H / G;
    const size_t smem = smem_bytes<true>();
    e = cudaFuncSetAttribute(attn_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((((int64_t)max_new * GS + 15) / 16) * n_splits, n_list, G);
    attn_mma_kernel<true><<<grid, THREADS, smem, stream>>>(a);
    SLLM_LAUNCH_CHECK();
    if (n_splits > 1) {
        dim3 mgrid(n_list, (H + MERGE_WARPS - 1) / MERGE_WARPS);
        attn_merge_kernel<<<mgrid, MERGE_WARPS * 32, 0, stream>>>(
            a.part_o, a.part_lse, n_splits, row_start, row_list, (bf16*)out, out_stride, H,
            a.part_tokens);
        SLLM_LAUNCH_CHECK();
    }
    return 0;
}
