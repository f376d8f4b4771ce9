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
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, temperature, top_p, seed,
                                                         counter, out, logprob_out, probs_out);
    SLLM_LAUNCH_CHECK();
    return 0;
}
