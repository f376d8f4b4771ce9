// sllm_attn_mma_split_noalloc: the split-KV decode attention for callers that must not
// allocate device memory.
//
// This entry point has no counterpart in the reference (andreidhoang/scratch_llm): its paged
// decode kernels take their partial-result buffers from the caller's PyTorch allocator.
//
// Who needs it.  sllm_attn_mma (attention_mma.cu) wants a scratch buffer for the per-split
// partial outputs and log-sum-exps, which its caller normally gets from cudaMalloc or from
// PyTorch's caching allocator.  Some callers cannot do that: a plug-in that runs inside another
// program's fixed device-memory budget and may not touch its allocator; a serving loop with a
// latency bound, where cudaMalloc may synchronise the whole device; code that has no PyTorch
// at all and drives the library through its C symbols.  For them the scratch lives in a
// file-scope `static __device__` array inside the library, of SLLM_NOALLOC_SCRATCH_FLOATS
// 32-bit floats (8 MiB).  Every GPU on which the library is loaded holds those 8 MiB until the
// process exits, used or not; one such array exists per compiled head size.
//
// Contract.
//  * Same arguments as sllm_attn_mma with split = 1, without `scratch`; inputs and outputs are
//    still the caller's.  Results equal sllm_attn_mma's up to bfloat16 rounding (for head
//    sizes that are multiples of 64 that entry point runs another kernel of the same math).
//  * n_tokens_total is the token count of the WHOLE batch that row_start describes: one past
//    the largest token index of any listed row (row_start[r + 1] for the last listed row r),
//    not the number of tokens in the listed rows.  Partial results are indexed by a token's
//    index in the batch.  A listed row that reaches beyond n_tokens_total is not written
//    outside the array: the tokens beyond it are left out of the output, and
//    sllm_attn_mma_noalloc_overrun() then returns 1.
//  * 1 <= n_splits <= SLLM_NOALLOC_MAX_SPLITS.
//  * Calls no cudaMalloc, cudaFree or any allocating library routine.
//  * Size limit: n_tokens_total * H * n_splits * (head size + 1) floats must fit the array
//    (n_splits = 1 needs none).  A larger request is refused: the call returns
//    cudaErrorInvalidValue (1), launches nothing, and sllm_attn_mma_noalloc_error() returns a
//    text that states the needed and the available size.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call
//    before any stream capture begins on that device.
//  * All calls share the one array and it keeps the previous call's contents.  Nothing in it
//    has to start at zero: every partial result that the merge step reads is written earlier
//    in the same call.  Two calls that overlap on the GPU (different streams, or different
//    host threads launching at once) race on the array and corrupt each other's results:
//    order them on one stream or with events.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifndef SLLM_NOALLOC_SCRATCH_FLOATS
#define SLLM_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#endif
#define SLLM_NOALLOC_MAX_SPLITS 1024

extern "C" {

// Returns 0 or a cudaError_t.  See attention_mma.cu::sllm_attn_mma for the tensor layouts.
int sllm_attn_mma_split_noalloc(const void* q, int64_t q_stride, const void* pages,
                                const int* block_table, int table_stride, int page_size,
                                const int* row_start, const int* row_pos0, const int* row_list,
                                int n_list, int max_new, void* out, int64_t out_stride, int H,
                                int G, float scale, int window, int n_splits,
                                int64_t n_tokens_total, cudaStream_t stream);

// The capacity of the built-in scratch array, in floats.
int64_t sllm_attn_mma_noalloc_capacity_floats(void);

// Text of the last refusal of sllm_attn_mma_split_noalloc in this process ("" if none).  One
// buffer per process, written without a lock: read it from the thread that got the refusal,
// before another thread calls the entry point.
const char* sllm_attn_mma_noalloc_error(void);

// 1 if a kernel of an earlier call on the current device met a token at or beyond its
// n_tokens_total (see above), 0 if none did, -1 if the flag could not be read.  Waits for the
// device (a copy from device memory) and clears the flag.
int sllm_attn_mma_noalloc_overrun(void);
}
