// Next-token choice on the device: greedy argmax, temperature sampling with the nucleus
// (top-p) filter, and the chosen token's log-probability.
//
// Restates src/scratch_llm/sampling.py:60-95 of the reference: temperature 0 takes the argmax
// (first maximum on ties); otherwise p = softmax(logits / T) with the maximum subtracted, the
// nucleus keeps the most probable tokens while the mass before a token is <= top_p (so the
// token that crosses top_p is kept), renormalises, and draws once.  The log-probability is
// log_softmax(raw logits)[token], at temperature 1.
//
// The reference draws from torch's global generator; here every request owns a counter-based
// generator (Philox-4x32-10 keyed by its seed, counter = how many tokens it has drawn), so a
// request's tokens do not depend on what else is in the batch.
//
// The nucleus needs no sort: token k is kept iff the mass of all strictly more probable
// tokens is <= top_p, which is monotone in p_k, so the smallest kept probability is found by
// bisection over float bit patterns (31 passes over the row, which stays in L2).
#include <cooperative_groups.h>

#include "common.cuh"

namespace sllm {

constexpr int SAMPLE_THREADS = 1024;

struct ArgMax {
    float v;
    int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    // larger value wins; on equal values the smaller index; an index of -1 is "nothing yet"
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        ArgMax t = lane < n_warps ? scratch[lane] : ArgMax{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax b;
            b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, b);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        float t = lane < n_warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
    const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// Uniform in [0, 1) from (seed, counter): Philox-4x32-10, first output word, top 24 bits.
__device__ float philox_uniform(unsigned long long seed, unsigned long long counter) {
    uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

// One block per row.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t ld, int V,
              const float* __restrict__ temperature, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seed,
              const unsigned long long* __restrict__ counter, int* __restrict__ out,
              float* __restrict__ logprob_out, float* __restrict__ probs_out) {
    __shared__ float fscratch[33];
    __shared__ ArgMax ascratch[33];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int chosen;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* z = logits + (int64_t)row * ld;
    const float T = temperature ? temperature[row] : 0.f;

    ArgMax best{0.f, -1};
    for (int i = tid; i < V; i += blockDim.x) best = better(best, ArgMax{z[i], i});
    best = block_argmax(best, ascratch);
    const float zmax = best.v;

    int token = best.i;
    if (T > 0.f) {
        const float inv_t = 1.0f / T;
        // softmax(z / T): the maximum of z / T is zmax / T for T > 0
        const float mt = zmax * inv_t;
        float part = 0.f;
        for (int i = tid; i < V; i += blockDim.x) part += expf(z[i] * inv_t - mt);
        const float Z = block_sum(part, fscratch);
        const float inv_z = 1.0f / Z;
        float thresh = 0.f;  // keep p >= thresh
        const float tp = top_p ? top_p[row] : 1.f;
        if (tp < 1.0f) {
            // f(t) = sum of p_i > t.  lo: f(lo) > tp.  hi: f(hi) <= tp.  p_max = 1 / Z.
            unsigned lo = 0u, hi = __float_as_uint(inv_z);
            while (hi - lo > 1u) {
                const unsigned mid = lo + (hi - lo) / 2u;
                const float t = __uint_as_float(mid);
                float above = 0.f;
                for (int i = tid; i < V; i += blockDim.x) {
                    const float p = expf(z[i] * inv_t - mt) * inv_z;
                    above += p > t ? p : 0.f;
                }
                above = block_sum(above, fscratch);
                if (above <= tp) hi = mid; else lo = mid;
            }
            thresh = __uint_as_float(hi);
        }
        // contiguous chunk per thread, in index order
        const int per = (V + blockDim.x - 1) / blockDim.x;
        const int begin = min(V, tid * per), end = min(V, begin + per);
        float mine = 0.f;
        for (int i = begin; i < end; ++i) {
            const float p = expf(z[i] * inv_t - mt) * inv_z;
            mine += p >= thresh ? p : 0.f;
        }
        chunk_sum[tid] = mine;
        const float kept = block_sum(mine, fscratch);
        if (probs_out) {
            float* po = probs_out + (int64_t)row * V;
            for (int i = tid; i < V; i += blockDim.x) {
                const float p = expf(z[i] * inv_t - mt) * inv_z;
                po[i] = p >= thresh ? p / kept : 0.f;
            }
        }
        if (tid == 0) chosen = -1;
        __syncthreads();
        const float u = philox_uniform(seed ? seed[row] : 0ull, counter ? counter[row] : 0ull);
        const float target = u * kept;
        // exclusive prefix of the chunk sums, by every thread for itself (1024 adds from
        // shared memory; once per sampled token)
        float before = 0.f;
        for (int t = 0; t < tid; ++t) before += chunk_sum[t];
        if (mine > 0.f && target >= before && target < before + mine) {
            float run = before;
            int pick = -1, last_kept = -1;
            for (int i = begin; i < end; ++i) {
                const float p = expf(z[i] * inv_t - mt) * inv_z;
                if (p >= thresh) {
                    last_kept = i;
                    run += p;
                    if (pick < 0 && target < run) pick = i;
                }
            }
            atomicMax(&chosen, pick >= 0 ? pick : last_kept);
        }
        __syncthreads();
        // rounding can leave the target past every chunk's end: take the most probable token
        token = chosen >= 0 ? chosen : best.i;
    }
    if (tid == 0) out[row] = token;
    if (logprob_out) {
        float part = 0.f;
        for (int i = tid; i < V; i += blockDim.x) part += expf(z[i] - zmax);
        const float Z1 = block_sum(part, fscratch);
        if (tid == 0) logprob_out[row] = z[token] - zmax - logf(Z1);
    }
}

// The same choice for large vocabularies: a thread-block cluster of SC_RANKS CTAs per row.
// With one CTA per row every pass over the row streams it from L2 into one SM with one load in
// flight per thread, and the nucleus needs up to 33 passes: 0.96 ms for a row of 128,256 logits,
// whatever the number of rows.  Here each CTA of the cluster keeps an eighth of the row in its
// shared memory (the logits, then the probabilities in their place), a pass is a
// walk over shared memory, and the CTAs add their partial results through distributed shared
// memory: every CTA writes its partial into a slot of every CTA, the cluster meets at its
// barrier, and each adds the eight slots in rank order, so that all hold the same bits and take
// the same branches.  (Two sets of slots take turns: a CTA can be one round ahead of another,
// never two.)  The bisection stops as soon as no probability lies strictly between its bounds:
// the threshold can then only be the upper one (22 rounds instead of 31 for 128,256 random
// logits; eight ways per round instead of two took 8 rounds but as long, a round's arithmetic
// growing as its number fell).  Arithmetic and rules are those of
// sample_kernel; only the order of the sums differs.
constexpr int SC_RANKS = 8;
constexpr int SC_MAX_SLICE = 24576;     // values a CTA keeps in shared memory (two CTAs share an SM)
constexpr int SC_MIN_VOCAB = 8192;      // below, one CTA per row has the row in L1 anyway

struct ScSlots {
    float f[2][SC_RANKS][2];
    ArgMax a[2][SC_RANKS];
    int i[2][SC_RANKS];
};

namespace cg = cooperative_groups;

// every CTA's (x, y) summed over the cluster, the same bits in every CTA
__device__ __forceinline__ float2 sc_all_sum(cg::cluster_group& cluster, ScSlots* slots, int& round,
                                             float x, float y) {
    const int set = round & 1;
    ++round;
    if (threadIdx.x < SC_RANKS) {
        ScSlots* peer = cluster.map_shared_rank(slots, threadIdx.x);
        peer->f[set][cluster.block_rank()][0] = x;
        peer->f[set][cluster.block_rank()][1] = y;
    }
    cluster.sync();
    float2 total = make_float2(0.f, 0.f);
#pragma unroll
    for (int r = 0; r < SC_RANKS; ++r) {
        total.x += slots->f[set][r][0];
        total.y += slots->f[set][r][1];
    }
    return total;
}


// N values per CTA summed over the block and then over the cluster (in v, the same bits in every
// thread of every CTA).  scratch: [32][N] floats.
template <int N>
__device__ __forceinline__ void sc_all_sum_n(cg::cluster_group& cluster, ScSlots* slots, int& round,
                                             float (&v)[N], float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = warp_sum(v[k]);
    __syncthreads();        // scratch may still be read from the round before
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < N; ++k) scratch[warp * N + k] = v[k];
    }
    __syncthreads();
    const int set = round & 1;
    ++round;
    if (threadIdx.x < SC_RANKS * N) {
        // thread (peer, k): the block's sum of value k, in warp order, into the peer's slot
        const int peer = threadIdx.x / N, k = threadIdx.x % N;
        float t = 0.f;
        for (int w = 0; w < SAMPLE_THREADS / 32; ++w) t += scratch[w * N + k];
        cluster.map_shared_rank(slots, peer)->f[set][cluster.block_rank()][k] = t;
    }
    cluster.sync();
#pragma unroll
    for (int k = 0; k < N; ++k) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < SC_RANKS; ++r) t += slots->f[set][r][k];
        v[k] = t;
    }
}

// NUCLEUS = false: no row has a top_p below 1 (top_p is not read); the kernel then needs few
// registers and two CTAs share an SM.
template <bool NUCLEUS>
__global__ void __cluster_dims__(SC_RANKS, 1, 1) __launch_bounds__(SAMPLE_THREADS, 2)
sample_cluster_kernel(const float* __restrict__ logits, int64_t ld, int V, int slice,
                      const float* __restrict__ temperature, const float* __restrict__ top_p,
                      const unsigned long long* __restrict__ seed,
                      const unsigned long long* __restrict__ counter, int* __restrict__ out,
                      float* __restrict__ logprob_out, float* __restrict__ probs_out) {
    extern __shared__ float sc_values[];       // [slice] logits, later their probabilities
    __shared__ float fscratch[33];
    __shared__ ArgMax ascratch[33];
    __shared__ float chunk_sum[32];
    __shared__ float nscratch[NUCLEUS ? 32 * 2 : 1];
    __shared__ int chosen;
    __shared__ ScSlots slots;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int row = blockIdx.x / SC_RANKS, tid = threadIdx.x;
    const float* z = logits + (int64_t)row * ld;
    const float T = temperature ? temperature[row] : 0.f;
    const int begin = min(V, rank * slice), n = min(V, begin + slice) - begin;
    float* zs = sc_values;      // the slice's logits until the probabilities take their place
    float* ps = sc_values;
    int round = 0;

    ArgMax best{0.f, -1};
    for (int i = tid; i < n; i += SAMPLE_THREADS) {
        const float v = z[begin + i];
        zs[i] = v;
        best = better(best, ArgMax{v, begin + i});
    }
    best = block_argmax(best, ascratch);
    {   // the row's first maximum: every CTA's candidate to every CTA
        const int set = round & 1;
        ++round;
        if (tid < SC_RANKS) cluster.map_shared_rank(&slots, tid)->a[set][rank] = best;
        cluster.sync();
        best = ArgMax{0.f, -1};
#pragma unroll
        for (int r = 0; r < SC_RANKS; ++r) best = better(best, slots.a[set][r]);
    }
    const float zmax = best.v;

    int token = best.i;
    if (T > 0.f) {     // (the same in every CTA of the cluster: they serve one row)
        const float inv_t = 1.0f / T;
        const float mt = zmax * inv_t;
        float part = 0.f;
        for (int i = tid; i < n; i += SAMPLE_THREADS) {
            const float e = expf(zs[i] * inv_t - mt);
            ps[i] = e;
            part += e;
        }
        const float Z = sc_all_sum(cluster, &slots, round, block_sum(part, fscratch), 0.f).x;
        const float inv_z = 1.0f / Z;
        for (int i = tid; i < n; i += SAMPLE_THREADS) ps[i] *= inv_z;
        __syncthreads();
        float thresh = 0.f;  // keep p >= thresh
        const float tp = NUCLEUS && top_p ? top_p[row] : 1.f;
        if (NUCLEUS && tp < 1.0f) {
            // f(t) = sum of p_i > t.  lo: f(lo) > tp.  hi: f(hi) <= tp.  p_max = 1 / Z.
            unsigned lo = 0u, hi = __float_as_uint(inv_z);
            while (hi - lo > 1u) {
                const unsigned mid = lo + (hi - lo) / 2u;
                const float t = __uint_as_float(mid);
                float v[2] = {0.f, 0.f};       // f(mid); how many probabilities lie inside
                for (int i = tid; i < n; i += SAMPLE_THREADS) {
                    const float p = ps[i];
                    v[0] += p > t ? p : 0.f;
                    const unsigned bits = __float_as_uint(p);
                    v[1] += (bits > lo && bits < hi && bits != mid) ? 1.f : 0.f;
                }
                sc_all_sum_n<2>(cluster, &slots, round, v, nscratch);
                if (v[0] <= tp) hi = mid; else lo = mid;
                // no probability strictly inside the bounds (mid has just become one of them):
                // f is constant on [lo, hi), so the search can only end at this hi
                if (v[1] == 0.f) break;
            }
            thresh = __uint_as_float(hi);
        }
        // contiguous chunk per thread, in index order; the CTAs' slices follow one another
        const int per = (n + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
        const int c0 = min(n, tid * per), c1 = min(n, c0 + per);
        float mine = 0.f;
        for (int i = c0; i < c1; ++i) {
            const float p = ps[i];
            mine += p >= thresh ? p : 0.f;
        }
        const float my_total = block_sum(mine, fscratch);
        const int set = round & 1;
        const float kept = sc_all_sum(cluster, &slots, round, my_total, 0.f).x;
        float before_cta = 0.f;
        for (int r = 0; r < rank; ++r) before_cta += slots.f[set][r][0];
        if (probs_out) {
            float* po = probs_out + (int64_t)row * V + begin;
            for (int i = tid; i < n; i += SAMPLE_THREADS) {
                const float p = ps[i];
                po[i] = p >= thresh ? p / kept : 0.f;
            }
        }
        if (tid == 0) chosen = -1;
        __syncthreads();
        const float u = philox_uniform(seed ? seed[row] : 0ull, counter ? counter[row] : 0ull);
        const float target = u * kept;
        // exclusive prefix of the chunk sums: the warps before this one (their totals, in warp
        // order), then the lanes before this one
        float before = before_cta;
        {
            const int lane = tid & 31, warp = tid >> 5;
            float incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (lane == 31) chunk_sum[warp] = incl;      // (chunk_sum is free: totals of the warps)
            __syncthreads();
            for (int w = 0; w < warp; ++w) before += chunk_sum[w];
            before += incl - mine;
        }
        if (mine > 0.f && target >= before && target < before + mine) {
            float run = before;
            int pick = -1, last_kept = -1;
            for (int i = c0; i < c1; ++i) {
                const float p = ps[i];
                if (p >= thresh) {
                    last_kept = begin + i;
                    run += p;
                    if (pick < 0 && target < run) pick = begin + i;
                }
            }
            atomicMax(&chosen, pick >= 0 ? pick : last_kept);
        }
        __syncthreads();
        {   // the CTA whose slice holds the target has chosen; all learn the token
            const int cset = round & 1;
            ++round;
            if (tid < SC_RANKS) cluster.map_shared_rank(&slots, tid)->i[cset][rank] = chosen;
            cluster.sync();
            int c = -1;
#pragma unroll
            for (int r = 0; r < SC_RANKS; ++r) c = max(c, slots.i[cset][r]);
            // rounding can leave the target past every chunk's end: take the most probable token
            token = c >= 0 ? c : best.i;
        }
    }
    if (rank == 0 && tid == 0) out[row] = token;
    if (logprob_out) {
        float part = 0.f;
        if (T > 0.f) {      // the logits have left shared memory
            for (int i = tid; i < n; i += SAMPLE_THREADS) part += expf(z[begin + i] - zmax);
        } else {
            for (int i = tid; i < n; i += SAMPLE_THREADS) part += expf(zs[i] - zmax);
        }
        const float Z1 = sc_all_sum(cluster, &slots, round, block_sum(part, fscratch), 0.f).x;
        if (rank == 0 && tid == 0) logprob_out[row] = z[token] - zmax - logf(Z1);
    }
    // nobody leaves while a peer may still write into its slots
    cluster.sync();
}

// Greedy choice for many rows at once: grid (ARGMAX_CHUNKS, rows).  Each block finds the
// argmax of its slice of the row; the block that finishes last for a row (a ticket from an
// atomic counter, no waiting) combines the slices.  `partial` holds ARGMAX_CHUNKS (value,
// index) pairs per row; `tickets` holds one counter per row, zero before the first call and
// reset to zero by the combining block.
constexpr int ARGMAX_CHUNKS = 32, ARGMAX_THREADS = 256;

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, int64_t ld, int V, ArgMax* __restrict__ partial,
              unsigned* __restrict__ tickets, int* __restrict__ out) {
    __shared__ ArgMax ascratch[33];
    __shared__ bool last;
    const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
    const float* z = logits + (int64_t)row * ld;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int begin = min(V, chunk * per), end = min(V, begin + per);
    ArgMax best{0.f, -1};
    for (int i = begin + tid; i < end; i += ARGMAX_THREADS) best = better(best, ArgMax{z[i], i});
    best = block_argmax(best, ascratch);
    if (tid == 0) {
        partial[row * ARGMAX_CHUNKS + chunk] = best;
        __threadfence();
        last = atomicAdd(&tickets[row], 1u) == ARGMAX_CHUNKS - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    ArgMax b = tid < ARGMAX_CHUNKS ? partial[row * ARGMAX_CHUNKS + tid] : ArgMax{0.f, -1};
    b = block_argmax(b, ascratch);
    if (tid == 0) {
        out[row] = b.i;
        tickets[row] = 0u;
    }
}

// log_softmax of each row in 32-bit (maximum subtracted, expf and logf at full precision).
// rows_out != nullptr: the whole row [n_rows, V]; taken != nullptr: taken_out[r] =
// log_softmax(logits[r])[taken[r]] (the log-probability of a given token, the reference's
// LocalBackend.score: src/scratch_llm/rollout/local.py:50-79).  One block per row.
__global__ void __launch_bounds__(SAMPLE_THREADS)
log_softmax_kernel(const float* __restrict__ logits, int64_t ld, int V,
                   float* __restrict__ rows_out, const int* __restrict__ taken,
                   float* __restrict__ taken_out) {
    __shared__ float fscratch[33];
    __shared__ float red[33];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* z = logits + (int64_t)row * ld;
    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, z[i]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < (int)((blockDim.x + 31) >> 5); ++w) mx = fmaxf(mx, red[w]);
    float part = 0.f;
    for (int i = tid; i < V; i += blockDim.x) part += expf(z[i] - mx);
    const float lz = mx + logf(block_sum(part, fscratch));
    if (rows_out) {
        float* o = rows_out + (int64_t)row * V;
        for (int i = tid; i < V; i += blockDim.x) o[i] = z[i] - lz;
    }
    if (taken && taken_out && tid == 0) {
        const int t = taken[row];
        taken_out[row] = (t >= 0 && t < V) ? z[t] - lz : __int_as_float(0x7fc00000);
    }
}

}  // namespace sllm

using namespace sllm;

// See log_softmax_kernel.  rows_out, or taken and taken_out, may be nullptr.
SLLM_EXPORT int sllm_log_softmax(const float* logits, int64_t ld, int n_rows, int V,
                                 float* rows_out, const int* taken, float* taken_out,
                                 cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || ld < V || (taken != nullptr) != (taken_out != nullptr))
        return (int)cudaErrorInvalidValue;
    log_softmax_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, rows_out, taken,
                                                              taken_out);
    SLLM_LAUNCH_CHECK();
    return 0;
}

// Bytes of scratch sllm_argmax needs for n_rows rows (partial results and tickets).  The
// tickets (the last 4 * n_rows bytes) must be zero before the first call.
SLLM_EXPORT int64_t sllm_argmax_scratch_bytes(int n_rows) {
    return (int64_t)n_rows * (ARGMAX_CHUNKS * (int64_t)sizeof(ArgMax) + 4);
}

// out[r] = index of the first maximum of logits[r, 0..V).
SLLM_EXPORT int sllm_argmax(const float* logits, int64_t ld, int n_rows, int V, void* scratch,
                            int* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || ld < V || n_rows > 65535 || !scratch) return (int)cudaErrorInvalidValue;
    ArgMax* partial = (ArgMax*)scratch;
    unsigned* tickets = (unsigned*)((char*)scratch + (int64_t)n_rows * ARGMAX_CHUNKS * sizeof(ArgMax));
    argmax_kernel<<<dim3(ARGMAX_CHUNKS, n_rows), ARGMAX_THREADS, 0, stream>>>(logits, ld, V, partial,
                                                                              tickets, out);
    SLLM_LAUNCH_CHECK();
    return 0;
}

// logits: [n_rows, ld] 32-bit, V columns used.  temperature == nullptr (or an entry 0) is
// greedy.  top_p / seed / counter / logprob_out / probs_out may be nullptr.
SLLM_EXPORT int sllm_sample(const float* logits, int64_t ld, int n_rows, int V,
                            const float* temperature, const float* top_p,
                            const unsigned long long* seed, const unsigned long long* counter,
                            int* out, float* logprob_out, float* probs_out,
                            cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || ld < V) return (int)cudaErrorInvalidValue;
    // large vocabularies: a cluster of CTAs per row, each with its slice in shared memory
    const int slice = ((V + SC_RANKS - 1) / SC_RANKS + 3) / 4 * 4;
    if (V >= SC_MIN_VOCAB && slice <= SC_MAX_SLICE) {
        const size_t smem = (size_t)slice * sizeof(float);
        auto kernel = top_p ? sample_cluster_kernel<true> : sample_cluster_kernel<false>;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        kernel<<<n_rows * SC_RANKS, SAMPLE_THREADS, smem, stream>>>(
            logits, ld, V, slice, temperature, top_p, seed, counter, out, logprob_out, probs_out);
        SLLM_LAUNCH_CHECK();
        return 0;
    }
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, temperature, top_p, seed,
                                                         counter, out, logprob_out, probs_out);
    SLLM_LAUNCH_CHECK();
    return 0;
}
