"""The decode attention entry point that allocates nothing (csrc/attention_mma_noalloc.h).

Some users of the kernel library cannot allocate device memory themselves: a plug-in living
inside another program's fixed memory budget, a loop that cannot afford cudaMalloc's device
synchronisation, or C code that has no PyTorch allocator at hand.  For them
``sllm_attn_mma_split_noalloc`` keeps the split-KV partial results in an array that is built
into the library.  This test calls that function through its exported C symbol, twice in a row
with different splits and inputs (the array keeps what the first call left in it), and checks
each output against the ordinary entry point, which is given scratch from PyTorch.

Collected last, so that a run that stops at the first failure has run every other test.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

H, G, HD, PAGE = 8, 2, 64, 16
CONTEXTS = [1, 63, 64, 65, 300, 1000]   # keys each decode row attends to (its own included)


def build_case(seed):
    g = torch.Generator().manual_seed(seed)
    n_rows = len(CONTEXTS)
    n_pages = sum(-(-c // PAGE) for c in CONTEXTS) + 2
    pages = (torch.randn(n_pages, 2, G, PAGE, HD, generator=g)).to(torch.bfloat16)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_rows, max(-(-c // PAGE) for c in CONTEXTS)), -1, dtype=torch.int32)
    for r, c in enumerate(CONTEXTS):
        for p in range(-(-c // PAGE)):
            table[r, p] = order.pop()
    q = torch.randn(n_rows, H * HD, generator=g).to(torch.bfloat16)
    row_start = torch.arange(n_rows + 1, dtype=torch.int32)
    row_pos0 = torch.tensor([c - 1 for c in CONTEXTS], dtype=torch.int32)
    return [t.cuda() for t in (q, pages, table, row_start, row_pos0)]


def call_noalloc(lib, q, pages, table, row_start, row_pos0, out, n_splits):
    ptr = lambda t: c_void_p(t.data_ptr())  # noqa: E731
    return lib.sllm_attn_mma_split_noalloc(
        ptr(q), c_int64(q.stride(0)), ptr(pages), ptr(table), c_int(table.stride(0)), c_int(PAGE),
        ptr(row_start), ptr(row_pos0), c_void_p(0), c_int(q.shape[0]), c_int(1), ptr(out),
        c_int64(out.stride(0)), c_int(H), c_int(G), c_float(1.0 / math.sqrt(HD)), c_int(0),
        c_int(n_splits), c_int64(q.shape[0]), c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_allocating_one():
    from scratch_llm_b200.kernels import build, ops

    lib = ctypes.CDLL(str(build.compile_library(*ops.attention_mma_library(HD), verbose=False)))
    lib.sllm_attn_mma_noalloc_capacity_floats.restype = c_int64
    lib.sllm_attn_mma_noalloc_error.restype = ctypes.c_char_p
    capacity = lib.sllm_attn_mma_noalloc_capacity_floats()
    assert capacity == 2 * 1024 * 1024

    for seed, n_splits in ((1, 8), (2, 3)):       # two calls in a row on the shared array
        q, pages, table, row_start, row_pos0 = build_case(seed)
        n = q.shape[0]
        want = torch.empty_like(q)
        scratch = torch.empty(ops.attention_mma_scratch_floats(n, H, HD, n_splits),
                              dtype=torch.float32, device="cuda")
        ops.attention_mma(q, pages, table, PAGE, row_start, row_pos0, want, None, n, 1, H, G, HD,
                          1.0 / math.sqrt(HD), None, split=True, n_splits=n_splits,
                          scratch=scratch)
        got = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_allocated()
        code = call_noalloc(lib, q, pages, table, row_start, row_pos0, got, n_splits)
        assert code == 0, lib.sllm_attn_mma_noalloc_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1e-2)
        assert torch.isfinite(got.float()).all()

    # a request beyond the built-in array is refused with a text that says why
    q, pages, table, row_start, row_pos0 = build_case(3)
    got = torch.zeros_like(q)
    too_many = capacity // (q.shape[0] * H * (HD + 1)) + 1
    code = call_noalloc(lib, q, pages, table, row_start, row_pos0, got, too_many)
    assert code == 1
    text = lib.sllm_attn_mma_noalloc_error().decode()
    assert "scratch floats" in text and str(capacity) in text
    assert not got.any()   # nothing was launched
