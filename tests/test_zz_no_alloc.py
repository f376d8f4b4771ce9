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


def call_noalloc(lib, q, pages, table, row_start, row_pos0, out, n_splits, row_list=None,
                 n_list=None, max_new=1, window=0, n_tokens_total=None):
    ptr = lambda t: c_void_p(t.data_ptr())  # noqa: E731
    return lib.sllm_attn_mma_split_noalloc(
        ptr(q), c_int64(q.stride(0)), ptr(pages), ptr(table), c_int(table.stride(0)), c_int(PAGE),
        ptr(row_start), ptr(row_pos0), ptr(row_list) if row_list is not None else c_void_p(0),
        c_int(q.shape[0] if n_list is None else n_list), c_int(max_new), ptr(out),
        c_int64(out.stride(0)), c_int(H), c_int(G), c_float(1.0 / math.sqrt(HD)), c_int(window),
        c_int(n_splits), c_int64(q.shape[0] if n_tokens_total is None else n_tokens_total),
        c_void_p(torch.cuda.current_stream().cuda_stream))


def load_library():
    from scratch_llm_b200.kernels import build, ops

    lib = ctypes.CDLL(str(build.compile_library(*ops.attention_mma_library(HD), verbose=False)))
    lib.sllm_attn_mma_noalloc_capacity_floats.restype = c_int64
    lib.sllm_attn_mma_noalloc_error.restype = ctypes.c_char_p
    return lib


def test_no_alloc_entry_point_matches_the_allocating_one():
    from scratch_llm_b200.kernels import ops

    lib = load_library()
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


# rows of a larger batch: (keys cached before this step, new tokens).  The call lists rows 1, 3
# and 4 only; their tokens lie in the middle and at the end of the batch.
ROWS = [(40, 5), (70, 3), (0, 9), (129, 1), (15, 2)]
LISTED = [1, 3, 4]
WINDOW = 37


def test_no_alloc_entry_point_with_a_row_list_several_tokens_and_a_window():
    """Listed rows of a larger batch, rows of several new tokens and a window of keys, against
    the plain attention; then the same call with a token count that covers only the listed
    rows' tokens (a caller's likely mistake): nothing is written outside the array, the tokens
    beyond the count are left out and the overrun flag says so."""
    from plain import llama_plain as P

    lib = load_library()
    g = torch.Generator().manual_seed(11)
    ks = [torch.randn(G, a + n, HD, generator=g).to(torch.bfloat16).float() for a, n in ROWS]
    vs = [torch.randn(G, a + n, HD, generator=g).to(torch.bfloat16).float() for a, n in ROWS]
    qs = [torch.randn(H, n, HD, generator=g).to(torch.bfloat16).float() for a, n in ROWS]
    n_pages = sum(-(-(a + n) // PAGE) for a, n in ROWS) + 1
    pages = torch.full((n_pages, 2, G, PAGE, HD), float("nan")).to(torch.bfloat16)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(ROWS), max(-(-(a + n) // PAGE) for a, n in ROWS)), -1,
                       dtype=torch.int32)
    for r, (k, v) in enumerate(zip(ks, vs)):
        for p in range(-(-k.shape[1] // PAGE)):
            phys = order.pop()
            table[r, p] = phys
            m = min(PAGE, k.shape[1] - p * PAGE)
            pages[phys, 0, :, :m] = k[:, p * PAGE:p * PAGE + m].to(torch.bfloat16)
            pages[phys, 1, :, :m] = v[:, p * PAGE:p * PAGE + m].to(torch.bfloat16)
    q = torch.cat([x.transpose(0, 1).reshape(x.shape[1], H * HD) for x in qs]).to(torch.bfloat16)
    starts = [0]
    for _, n in ROWS:
        starts.append(starts[-1] + n)
    dev = [t.cuda() for t in (q, pages, table, torch.tensor(starts, dtype=torch.int32),
                              torch.tensor([a for a, _ in ROWS], dtype=torch.int32),
                              torch.tensor(LISTED, dtype=torch.int32))]
    q, pages, table, row_start, row_pos0, row_list = dev
    max_new = max(ROWS[r][1] for r in LISTED)

    def plain_row(r):
        a, n = ROWS[r]
        out = P.attention(qs[r], ks[r], vs[r], torch.arange(a, a + n), torch.arange(a + n),
                          1.0 / math.sqrt(HD), WINDOW)
        return out.transpose(0, 1).reshape(n, H * HD)

    for n_splits in (4, 1):
        got = torch.full_like(q, float("nan"))
        code = call_noalloc(lib, q, pages, table, row_start, row_pos0, got, n_splits,
                            row_list=row_list, n_list=len(LISTED), max_new=max_new, window=WINDOW)
        assert code == 0, lib.sllm_attn_mma_noalloc_error()
        torch.cuda.synchronize()
        assert lib.sllm_attn_mma_noalloc_overrun() == 0
        got = got.cpu().float()
        for r in range(len(ROWS)):
            mine = got[starts[r]:starts[r + 1]]
            if r in LISTED:
                torch.testing.assert_close(mine, plain_row(r), rtol=1.6e-2, atol=1e-2)
            else:
                assert torch.isnan(mine).all()   # rows that were not listed are not touched

    # a token count that covers only the listed rows' tokens (6) while their indices reach 20
    listed_tokens = sum(ROWS[r][1] for r in LISTED)
    got = torch.full_like(q, float("nan"))
    code = call_noalloc(lib, q, pages, table, row_start, row_pos0, got, 4, row_list=row_list,
                        n_list=len(LISTED), max_new=max_new, window=WINDOW,
                        n_tokens_total=listed_tokens)
    assert code == 0
    torch.cuda.synchronize()
    assert lib.sllm_attn_mma_noalloc_overrun() == 1
    assert lib.sllm_attn_mma_noalloc_overrun() == 0        # reading the flag clears it
    got = got.cpu().float()
    r = LISTED[0]                                           # tokens 5, 6, 7: index 5 is covered
    torch.testing.assert_close(got[5:6], plain_row(r)[:1], rtol=1.6e-2, atol=1e-2)
    assert torch.isnan(got[listed_tokens:]).all()           # the rest was left out, not written

    # out-of-range split counts are refused before anything is computed from them
    for bad in (0, 1025, 1 << 30):
        assert call_noalloc(lib, q, pages, table, row_start, row_pos0, got.cuda().bfloat16(), bad,
                            row_list=row_list, n_list=len(LISTED), max_new=max_new) == 1
