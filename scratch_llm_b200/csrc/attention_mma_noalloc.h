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
//  * Same arguments and results as sllm_attn_mma with split = 1, without `scratch`; inputs
//    and outputs are still the caller's.
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

// Text of the last refusal of sllm_attn_mma_split_noalloc in this process ("" if none).
const char* sllm_attn_mma_noalloc_error(void);
}
