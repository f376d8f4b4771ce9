"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's."""

import math

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(rtol=1e-5, atol=1e-6), "bfloat16": dict(rtol=1.6e-2, atol=1e-2)}


@pytest.fixture(scope="module")
def ops():
    from scratch_llm_b200.kernels import ops
    ops.prepare([16, 48, 80, 128], verbose=False)
    return ops


def rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("v", [331, 128256])
def test_log_softmax(ops, v):
    logits = rand(5, v + 3, seed=v, scale=4.0)[:, :v]          # rows inside a wider buffer
    logits[2, 7] = 60.0                                        # one token takes all the mass
    taken = torch.tensor([0, v - 1, 7, 123, 5], dtype=torch.int32)
    want = torch.log_softmax(logits.double(), dim=-1).float()
    x = logits.cuda()
    x = torch.cat([x, torch.zeros(5, 3, device="cuda")], 1)[:, :v]
    rows = torch.empty(5, v, dtype=torch.float32, device="cuda")
    lp = torch.empty(5, dtype=torch.float32, device="cuda")
    ops.log_softmax(x, rows_out=rows, taken=taken.cuda(), taken_out=lp)
    torch.testing.assert_close(rows.cpu(), want, rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(lp.cpu(), want[torch.arange(5), taken.long()], rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(ops, dtype):
    table = rand(1000, 200, dtype=DT[dtype])
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32)
    out = torch.empty(5, 200, dtype=torch.float32, device="cuda")
    ops.embed(ids.cuda(), table.cuda(), out)
    assert torch.equal(out.cpu(), P.embed(ids.long(), table).float())
    ops.embed(ids.cuda(), table.cuda(), out, scale=200 ** 0.5)
    assert torch.equal(out.cpu(), P.embed(ids.long(), table).float() * torch.tensor(200 ** 0.5))


@pytest.mark.parametrize("n, d, scale", [(8, 1024, 1.0), (3, 200, 2.5), (1, 4096, 1.0)])
def test_embed_prepares_the_first_norm(ops, n, d, scale):
    """The embedding for a few tokens that also writes the first norm's input for the product
    after it (stream * gain in bfloat16) and the tokens' sums of squares in groups of 8."""
    table = rand(500, d, dtype=torch.bfloat16, seed=1)
    gain = rand(d, seed=2) * 0.2 + 1.0
    ids = torch.tensor([499, 0, 7, 7, 123, -1, 42, 3][:n], dtype=torch.int32)
    pending = torch.tensor([321, 5], dtype=torch.int32)
    real = ids.clone().long()
    real[ids < 0] = 321
    out = torch.full((n, d), float("nan"), dtype=torch.float32, device="cuda")
    x_out = torch.full((n, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    shares = torch.full((d // 8, 8), float("nan"), dtype=torch.float32, device="cuda")
    ops.embed_prepare(ids.cuda(), table.cuda(), out, pending.cuda(), scale, gain.cuda(), x_out, shares)
    want = table[real].float() * scale
    assert torch.equal(out.cpu(), want)
    assert torch.equal(x_out.cpu(), (want * gain).to(torch.bfloat16))
    torch.testing.assert_close(shares.cpu()[:, :n].sum(0), want.pow(2).sum(-1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(shares.cpu()[:, :n].T.reshape(n, d // 8),
                               want.pow(2).reshape(n, d // 8, 8).sum(-1), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("scale, cap", [(1.0, 30.0), (0.25, 0.0), (3.0, 1.5)])
def test_logit_cap(ops, scale, cap):
    x = rand(7, 1001, seed=4) * 20
    got = ops.logit_cap(x.cuda().clone(), scale, cap).cpu()
    want = cap * torch.tanh(x * scale / cap) if cap else x * scale
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d, eps", [(4096, 1e-5), (120, 1e-6), (7, 1e-3), (5000, 1e-5)])
def test_add_rmsnorm(ops, dtype, d, eps):
    n = 9
    resid, delta = rand(n, d, seed=1), rand(n, d, dtype=DT[dtype], seed=2)
    w = rand(d, seed=3) + 1.0
    want_resid = resid + delta.float()
    want = P.rmsnorm(want_resid, w, eps)
    r = resid.cuda()
    out = torch.empty(n, d, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(r, delta.cuda(), w.cuda(), eps, out)
    torch.testing.assert_close(r.cpu(), want_resid, rtol=0, atol=0)
    torch.testing.assert_close(out.cpu().float(), want, **TOL[dtype])
    # without a delta the stream is left alone
    r2 = resid.cuda()
    ops.add_rmsnorm(r2, None, w.cuda(), eps, out)
    assert torch.equal(r2.cpu(), resid)
    torch.testing.assert_close(out.cpu().float(), P.rmsnorm(resid, w, eps), **TOL[dtype])
    # gathered rows: only those rows, delta added on the fly, stream untouched
    idx = torch.tensor([7, 0, 7, 3], dtype=torch.int32)
    r3 = resid.cuda()
    out4 = torch.empty(4, d, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(r3, delta.cuda(), w.cuda(), eps, out4, idx.cuda())
    assert torch.equal(r3.cpu(), resid)
    torch.testing.assert_close(out4.cpu().float(), want[idx.long()], **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [4096, 1000, 520])
def test_add_rmsnorm_same_bits_for_few_and_many_rows(ops, dtype, d):
    """With many rows the norm runs in narrower blocks; a row's result is bitwise the one it
    has among few rows (the sums are added in the same order)."""
    n = 400
    resid, delta = rand(n, d, seed=4), rand(n, d, dtype=DT[dtype], seed=5)
    w = rand(d, seed=6) + 1.0
    many_r, few_r = resid.cuda(), resid[:5].cuda()
    many = torch.empty(n, d, dtype=DT[dtype], device="cuda")
    few = torch.empty(5, d, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(many_r, delta.cuda(), w.cuda(), 1e-5, many)
    ops.add_rmsnorm(few_r, delta[:5].cuda(), w.cuda(), 1e-5, few)
    assert torch.equal(many.cpu()[:5], few.cpu()) and torch.equal(many_r.cpu()[:5], few_r.cpu())
    torch.testing.assert_close(many.cpu().float(), P.rmsnorm(resid + delta.float(), w, 1e-5),
                               **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(ops, dtype):
    gu = rand(13, 2 * 301, dtype=DT[dtype], scale=3.0)
    out = torch.empty(13, 301, dtype=DT[dtype], device="cuda")
    ops.swiglu(gu.cuda(), out)
    g, u = gu.float()[:, :301], gu.float()[:, 301:]
    torch.testing.assert_close(out.cpu().float(), g * torch.sigmoid(g) * u, **TOL[dtype])


@pytest.mark.parametrize("m, n, k", [(1, 100, 64), (70, 130, 200), (64, 64, 16), (3, 5, 7),
                                     (129, 257, 33)])
def test_gemm_simt_is_true_32_bit(ops, m, n, k):
    x, w = rand(m, k, seed=1), rand(n, k, seed=2)
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.gemm_simt(x.cuda(), w.cuda(), out)
    want = (x.double() @ w.double().T)
    # a tf32 product would be wrong by ~1e-3 relative; 32-bit accumulation by ~1e-6
    torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    # a row's result does not depend on the other rows of the batch: bitwise
    one = torch.empty(1, n, dtype=torch.float32, device="cuda")
    ops.gemm_simt(x[m // 2:m // 2 + 1].cuda(), w.cuda(), one)
    assert torch.equal(one.cpu()[0], out.cpu()[m // 2])


def test_gemm_simt_bfloat16_inputs(ops):
    x, w = rand(17, 96, dtype=torch.bfloat16, seed=1), rand(50, 96, dtype=torch.bfloat16, seed=2)
    out = torch.empty(17, 50, dtype=torch.float32, device="cuda")
    ops.gemm_simt(x.cuda(), w.cuda(), out)
    torch.testing.assert_close(out.cpu(), x.float() @ w.float().T, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("m, n, k", [(1, 16, 64), (3, 100, 200), (8, 4096 + 8, 4096), (9, 130, 264),
                                     (16, 512, 14336), (17, 96, 1000), (33, 260, 520),
                                     (64, 1024, 4096), (5, 7, 8)])
def test_gemv_streams_weights_once(ops, m, n, k):
    x = rand(m, k, dtype=torch.bfloat16, seed=1)
    w = rand(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.float() @ w.float().T
    for dt in (torch.float32, torch.bfloat16):
        out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        ops.gemv_mma(x.cuda(), w.cuda(), out)
        tol = dict(rtol=2e-3, atol=2e-3) if dt == torch.float32 else TOL["bfloat16"]
        torch.testing.assert_close(out.cpu().float(), want, **tol)
    # a token's result does not depend on its neighbours, nor on how many there are: bitwise
    full = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.gemv_mma(x.cuda(), w.cuda(), full)
    one = torch.empty(1, n, dtype=torch.float32, device="cuda")
    ops.gemv_mma(x[m - 1:].cuda(), w.cuda(), one)
    assert torch.equal(one.cpu()[0], full.cpu()[m - 1])
    if n % 2 == 0:
        half = n // 2
        out = torch.full((m, half), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemv_mma(x.cuda(), w.cuda(), out, swiglu=True)
        gate, up = want[:, :half].to(torch.bfloat16).float(), want[:, half:].to(torch.bfloat16).float()
        torch.testing.assert_close(out.cpu().float(), gate * torch.sigmoid(gate) * up,
                                   **TOL["bfloat16"])


@pytest.mark.parametrize("m, n, k", [(1, 16, 1024), (3, 100, 1536), (8, 4096 + 8, 4096),
                                     (5, 512, 14336), (8, 6144, 4096), (2, 44, 5120),
                                     (7, 9000, 2048), (4, 40000, 1024), (4, 1004, 13824),
                                     (8, 5120 * 3, 5120)])
def test_gemv_persistent_bulk_copies(ops, m, n, k):
    """The persistent small-batch product (weights through shared memory by bulk copies, ranges
    of K combined through words in global memory): values, launches in a row on the shared
    workspace, bitwise independence of the number of tokens, and the fused SwiGLU."""
    assert ops.gemv_tma_supports(m, n, k)
    assert not ops.gemv_tma_supports(9, n, k) and not ops.gemv_tma_supports(m, n, k + 8)
    x = rand(m, k, dtype=torch.bfloat16, seed=1)
    w = rand(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.float() @ w.float().T
    for dt in (torch.float32, torch.bfloat16):
        for _ in range(3):   # the words of the exchange are back at zero after every launch
            out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
            ops.gemv_tma(x.cuda(), w.cuda(), out)
            tol = dict(rtol=2e-3, atol=2e-3) if dt == torch.float32 else TOL["bfloat16"]
            torch.testing.assert_close(out.cpu().float(), want, **tol)
    full = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.gemv_tma(x.cuda(), w.cuda(), full)
    one = torch.empty(1, n, dtype=torch.float32, device="cuda")
    ops.gemv_tma(x[m - 1:].cuda(), w.cuda(), one)
    assert torch.equal(one.cpu()[0], full.cpu()[m - 1])
    if n % 2 == 0:
        half = n // 2
        out = torch.full((m, half), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemv_tma(x.cuda(), w.cuda(), out, swiglu=True)
        gate, up = want[:, :half].to(torch.bfloat16).float(), want[:, half:].to(torch.bfloat16).float()
        torch.testing.assert_close(out.cpu().float(), gate * torch.sigmoid(gate) * up,
                                   **TOL["bfloat16"])
    # rows of x and w inside wider buffers
    xw = torch.zeros(m, k + 64, dtype=torch.bfloat16)
    xw[:, :k] = x
    ww = torch.zeros(n, k + 8, dtype=torch.bfloat16)
    ww[:, :k] = w
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.gemv_tma(xw.cuda()[:, :k], ww.cuda()[:, :k], out)
    assert torch.equal(out.cpu(), full.cpu())
    assert ops.gemv_tma_error() == 0


@pytest.mark.parametrize("m, d, f, eps", [(8, 1024, 1536, 1e-5), (3, 4096, 2560, 1e-6),
                                          (1, 2048, 4608, 1e-3), (5, 1536, 1024, 1e-5)])
def test_gemv_hands_the_norm_over(ops, m, d, f, eps):
    """The two halves of a deferred RMS norm around the residual stream.  A product that ends a
    branch (f -> d) adds its output into the 32-bit stream, writes stream * gain and the
    tokens' shares of squares; the product that starts the next branch (d -> f, plain and with
    the fused activation) multiplies its outputs by rsqrt(mean(stream^2) + eps).  Together they
    must give what add + norm + product give in the plain order (src/scratch_llm/model.py:
    158-162, 430-435 of the reference)."""
    x = rand(m, f, dtype=torch.bfloat16, seed=1)
    w_end = rand(d, f, dtype=torch.bfloat16, seed=2, scale=0.05)
    w_next = rand(2 * f, d, dtype=torch.bfloat16, seed=3, scale=0.05)
    gain = rand(d, seed=4) * 0.2 + 1.0
    resid0 = rand(m + 2, d, seed=5, scale=3.0)        # two rows more: they must stay untouched
    # plain order
    y = (x.float() @ w_end.float().T).to(torch.bfloat16).float()
    stream = resid0[:m] + y
    normed = P.rmsnorm(stream, gain, eps)
    want_plain = normed @ w_next.float().T
    g, u = want_plain[:, :f].to(torch.bfloat16).float(), want_plain[:, f:].to(torch.bfloat16).float()
    want_act = g * torch.sigmoid(g) * u
    # the engine's order
    resid = resid0.cuda()
    x_out = torch.full((m, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    shares = torch.full((-(-d // 8), 8), float("nan"), dtype=torch.float32, device="cuda")
    ops.gemv_tma(x.cuda(), w_end.cuda(), None, sink=(resid[:m], gain.cuda(), x_out, shares))
    # (the product's output is rounded to bfloat16 before it is added, as the unfused path
    # does: a sum that lands on a tie may round the other way, one bfloat16 step of y)
    torch.testing.assert_close(resid.cpu()[:m], stream, rtol=0, atol=2.0 ** -7 * float(y.abs().max()))
    assert float((resid.cpu()[:m] - stream).abs().mean()) < 1e-5
    assert torch.equal(resid.cpu()[m:], resid0[m:])
    torch.testing.assert_close(x_out.cpu().float(), (stream * gain).to(torch.bfloat16).float(),
                               rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(shares.cpu()[:, :m].sum(0), stream.pow(2).sum(-1), rtol=1e-4, atol=1e-3)
    out = torch.full((m, 2 * f), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemv_tma(x_out, w_next.cuda(), out, scale=(shares, d, eps))
    # (activations rounded to bfloat16 once, before the factor instead of after it: errors of
    # a bfloat16 step of the inputs, measured against the largest output)
    torch.testing.assert_close(out.cpu().float(), want_plain, rtol=1.6e-2,
                               atol=1e-2 * float(want_plain.abs().max()))
    act = torch.full((m, f), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemv_tma(x_out, w_next.cuda(), act, swiglu=True, scale=(shares, d, eps))
    torch.testing.assert_close(act.cpu().float(), want_act, rtol=3e-2,
                               atol=1e-2 * float(want_act.abs().max()))
    # one token alone gives the bits it gave in the batch (sink and scale are per token)
    resid1 = resid0[m - 1:m].clone().cuda()
    x1 = torch.empty((1, d), dtype=torch.bfloat16, device="cuda")
    s1 = torch.empty_like(shares)
    ops.gemv_tma(x[m - 1:].cuda(), w_end.cuda(), None, sink=(resid1, gain.cuda(), x1, s1))
    o1 = torch.empty((1, 2 * f), dtype=torch.bfloat16, device="cuda")
    ops.gemv_tma(x1, w_next.cuda(), o1, scale=(s1, d, eps))
    assert torch.equal(o1.cpu()[0], out.cpu()[m - 1])
    assert ops.gemv_tma_error() == 0


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (128, 256, 256), (256, 512, 192), (300, 600, 200),
                                     (5, 40, 72), (2048, 1024, 512), (130, 6144, 4096),
                                     (513, 2560, 1024)])
@pytest.mark.parametrize("pairs", [True, False])
def test_gemm_tcgen05(ops, m, n, k, pairs):
    """Both kernels: tiles of 256 x 256 on pairs of SMs (cta_group::2), and tiles of 128 x 256 on
    single SMs."""
    ops.gemm_tc_set_pairs(pairs)
    try:
        _gemm_tcgen05_case(ops, m, n, k)
    finally:
        ops.gemm_tc_set_pairs(True)


@pytest.mark.parametrize("tile", [128, 112, 96, 80, 64, 48, 16])
@pytest.mark.parametrize("m, n, k", [(300, 600, 200), (256, 2 * 112 * 3, 256), (513, 2560, 1024),
                                     (40, 2 * 1000, 136)])
def test_gemm_tcgen05_gate_up_tile_widths(ops, m, n, k, tile):
    """The fused gate/up product on SM pairs with tiles of every width (features per tile): the
    gate and up halves of a tile sit side by side in tensor memory at the tile's width, a last
    chunk may hold 16 features, the last tile of a row of tiles may be cut by the matrix."""
    ops.gemm_tc_set_tile(tile)
    try:
        assert ops.gemm_tc_swiglu_tile(m, n // 2, 74) == tile
        _gemm_tcgen05_case(ops, m, n, k)
    finally:
        ops.gemm_tc_set_tile(None)


def test_gemm_tcgen05_tile_choice(ops):
    """The launcher's choice of a tile width: 112 features where that needs no more rounds of
    tiles than 128."""
    pick = ops.gemm_tc_swiglu_tile
    assert pick(1024, 14336, 74) == 112      # 448 or 512 tiles on 74 pairs: 7 rounds either way
    assert pick(2048, 14336, 74) == 128      # 13 rounds of 128, 14 of 112
    assert pick(2048, 8192, 74) == 128       # 7 rounds of 128, 8 of 112
    assert pick(448, 8192, 74) == 112        # 2 rounds either way
    assert pick(512, 13824, 74) == 128       # 3 rounds of 128, 4 of 112


def _gemm_tcgen05_case(ops, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    if k <= 256:   # small integers: every product and sum is exact, also in bfloat16
        x = torch.randint(-1, 2, (m, k), generator=g).to(torch.bfloat16)
        w = torch.randint(-1, 2, (n, k), generator=g).to(torch.bfloat16)
        tol = dict(rtol=0, atol=0)
    else:
        x = rand(m, k, dtype=torch.bfloat16, seed=1)
        w = rand(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
        tol = TOL["bfloat16"]
    want = x.float() @ w.float().T
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(x.cuda(), w.cuda(), out)
    assert ops.gemm_tc_error() == 0
    torch.testing.assert_close(out.cpu().float(), want.to(torch.bfloat16).float(), **tol)
    if n % 2 == 0:
        half = n // 2
        out = torch.full((m, half), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemm_tc(x.cuda(), w.cuda(), out, swiglu=True)
        assert ops.gemm_tc_error() == 0
        gate, up = want[:, :half].to(torch.bfloat16).float(), want[:, half:].to(torch.bfloat16).float()
        torch.testing.assert_close(out.cpu().float(), gate * torch.sigmoid(gate) * up,
                                   **TOL["bfloat16"])


def paged_cache(k, v, page_size, n_pages, seed, dtype):
    """Scatter k, v [G, T, hd] of several rows into shuffled pages.  Returns pages, tables."""
    g = torch.Generator().manual_seed(seed)
    G, hd = k[0].shape[0], k[0].shape[2]
    pages = torch.full((n_pages, 2, G, page_size, hd), float("nan")).to(dtype)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-kk.shape[1] // page_size) for kk in k)
    table = torch.full((len(k), width), -1, dtype=torch.int32)
    for r, (kk, vv) in enumerate(zip(k, v)):
        for p in range(-(-kk.shape[1] // page_size)):
            phys = order.pop()
            table[r, p] = phys
            n = min(page_size, kk.shape[1] - p * page_size)
            pages[phys, 0, :, :n] = kk[:, p * page_size:p * page_size + n].to(dtype)
            pages[phys, 1, :, :n] = vv[:, p * page_size:p * page_size + n].to(dtype)
    return pages, table


ATTN_SHAPES = [(4, 2, 16, 16, None), (6, 3, 48, 8, None), (8, 1, 128, 32, None),
               (5, 5, 80, 4, None), (4, 2, 16, 16, 37), (6, 2, 48, 8, 5), (40, 2, 16, 16, None),
               (8, 2, 64, 16, 37), (6, 3, 128, 8, 70), (4, 2, 192, 16, None)]
# rows: (cached before this step, new tokens): a whole prompt, portions, single tokens
ATTN_ROWS = [(0, 70), (33, 1), (64, 18), (100, 2), (0, 1), (255, 1), (17, 47), (63, 1), (64, 1)]
FAR = 5  # the row with 255 cached keys


def attention_case(dtype, H, G, hd, page):
    dt = DT[dtype]
    rows = ATTN_ROWS
    ks = [rand(G, a + n, hd, seed=10 + i).to(dt).float() for i, (a, n) in enumerate(rows)]
    vs = [rand(G, a + n, hd, seed=50 + i).to(dt).float() for i, (a, n) in enumerate(rows)]
    qs = [rand(H, n, hd, seed=90 + i).to(dt).float() for i, (a, n) in enumerate(rows)]
    # a far key among hundreds: key 3 of kv head 0 points along the query of head 0 and is
    # scaled so that its score stands out
    ks[FAR][0, 3] = qs[FAR][0, 0] / qs[FAR][0, 0].norm() * 12.0
    ks[FAR] = ks[FAR].to(dt).float()
    n_pages = sum(-(-(a + n) // page) for a, n in rows) + 3
    pages, table = paged_cache(ks, vs, page, n_pages, seed=7, dtype=dt)
    # unused places of the pages hold NaN: nothing may read them into a result
    q_flat = torch.cat([q.transpose(0, 1).reshape(q.shape[1], H * hd) for q in qs]).to(dt)
    wide = torch.zeros(q_flat.shape[0], H * hd + 64, dtype=dt)  # q inside a wider buffer
    wide[:, :H * hd] = q_flat
    row_start = torch.tensor([0] + list(torch.tensor([n for _, n in rows]).cumsum(0)),
                             dtype=torch.int32)
    row_pos0 = torch.tensor([a for a, _ in rows], dtype=torch.int32)
    return dict(qs=qs, ks=ks, vs=vs, pages=pages.cuda(), table=table.cuda(), wide=wide.cuda(),
                row_start=row_start.cuda(), row_pos0=row_pos0.cuda(), starts=row_start.tolist())


def check_attention(case, got, rows_checked, dtype, H, hd, window):
    scale = 1.0 / math.sqrt(hd)
    for i in rows_checked:
        a, n = ATTN_ROWS[i]
        t = case["starts"][i]
        want = P.attention(case["qs"][i], case["ks"][i], case["vs"][i], torch.arange(a, a + n),
                           torch.arange(a + n), scale, window)
        want = want.transpose(0, 1).reshape(n, H * hd)
        torch.testing.assert_close(got[t:t + n], want, **TOL[dtype],
                                   msg=lambda m: f"row {i} {ATTN_ROWS[i]}: {m}")
    if window is None and FAR in rows_checked:
        # the far key took nearly all the weight of head 0 in its row
        torch.testing.assert_close(got[case["starts"][FAR], :hd], case["vs"][FAR][0, 3],
                                   rtol=0.05, atol=0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, hd, page, window", ATTN_SHAPES)
def test_attention_over_pages(ops, dtype, H, G, hd, page, window):
    case = attention_case(dtype, H, G, hd, page)
    out = torch.full((case["wide"].shape[0], H * hd), float("nan"), dtype=DT[dtype], device="cuda")
    ops.attention_simt(case["wide"][:, :H * hd], case["pages"], case["table"], page,
                       case["row_start"], case["row_pos0"], out, len(ATTN_ROWS),
                       max(n for _, n in ATTN_ROWS), H, G, hd, 1.0 / math.sqrt(hd), window)
    check_attention(case, out.cpu().float(), range(len(ATTN_ROWS)), dtype, H, hd, window)


@pytest.mark.parametrize("n_splits", [1, 3, 8])
@pytest.mark.parametrize("H, G, hd, page, window", ATTN_SHAPES)
def test_attention_on_tensor_cores(ops, H, G, hd, page, window, n_splits):
    """The wide kernel on the rows with several new tokens, the split kernel on the rows with
    one; then each kernel on all rows (either takes any row)."""
    case = attention_case("bfloat16", H, G, hd, page)
    q = case["wide"][:, :H * hd]
    n_tok = q.shape[0]
    single = [i for i, (_, n) in enumerate(ATTN_ROWS) if n == 1]
    multi = [i for i, (_, n) in enumerate(ATTN_ROWS) if n > 1]
    every = list(range(len(ATTN_ROWS)))
    scale = 1.0 / math.sqrt(hd)
    scratch = torch.full((ops.attention_mma_scratch_floats(n_tok, H, hd, n_splits) + 1,),
                         float("nan"), dtype=torch.float32, device="cuda")
    base = (q, case["pages"], case["table"], page, case["row_start"], case["row_pos0"])
    for wide_rows, split_rows in ((multi, single), (every, []), ([], every)):
        out = torch.full((n_tok, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        if wide_rows:
            ops.attention_mma(*base, out, torch.tensor(wide_rows, dtype=torch.int32).cuda(),
                              len(wide_rows), max(ATTN_ROWS[i][1] for i in wide_rows), H, G, hd,
                              scale, window, split=False)
        if split_rows:
            ops.attention_mma(*base, out, torch.tensor(split_rows, dtype=torch.int32).cuda(),
                              len(split_rows), max(ATTN_ROWS[i][1] for i in split_rows), H, G, hd,
                              scale, window, split=True, n_splits=n_splits, scratch=scratch)
        check_attention(case, out.cpu().float(), every, "bfloat16", H, hd, window)


@pytest.mark.parametrize("n_splits", [1, 3, 8])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("H, G, hd, page, window", [(8, 2, 64, 16, None), (32, 8, 128, 64, None),
                                                    (6, 3, 128, 8, 70), (16, 1, 64, 16, None)])
def test_decode_attention_fused_with_rotation(ops, H, G, hd, page, window, n_splits, interleaved):
    """The decode kernel that takes q, k and v as the projection left them (rotates q and the new
    key, stores key and value) gives, bit for bit, what the separate kernels give (rotation and
    store, then split attention), and leaves the same cache."""
    import math
    contexts = [0, 1, 15, 16, 63, 64, 200, 517]          # keys cached before the step
    n = len(contexts)
    max_pos = 600
    cos, sin = P.rope_tables(hd, max_pos, 10000.0)
    per = [-(-(c + 1) // page) for c in contexts]
    n_pages = sum(per) + 2
    g = torch.Generator().manual_seed(3)
    pages = (torch.randn(n_pages, 2, G, page, hd, generator=g) * 0.5).to(torch.bfloat16)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n, max(per)), -1, dtype=torch.int32)
    for r in range(n):
        for p in range(per[r]):
            table[r, p] = order.pop()
    qkv = (torch.randn(n, (H + 2 * G) * hd, generator=g)).to(torch.bfloat16)
    row_start = torch.arange(n + 1, dtype=torch.int32).cuda()
    row_pos0 = torch.tensor(contexts, dtype=torch.int32).cuda()
    rows = torch.arange(n, dtype=torch.int32).cuda()
    scale = 1.0 / math.sqrt(hd)
    scratch = torch.empty(ops.attention_mma_scratch_floats(n, H, hd, n_splits) + 1,
                          dtype=torch.float32, device="cuda")
    # the separate kernels
    qkv_a, pages_a = qkv.clone().cuda(), pages.clone().cuda()
    ops.rope_kv_write(qkv_a, row_pos0, rows, cos.cuda(), sin.cuda(), pages_a, table.cuda(), page,
                      H, G, hd, interleaved, True)
    out_a = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention_mma(qkv_a[:, :H * hd], pages_a, table.cuda(), page, row_start, row_pos0, out_a,
                      rows, n, 1, H, G, hd, scale, window, split=True, n_splits=n_splits,
                      scratch=scratch)
    # the one kernel
    pages_b = pages.clone().cuda()
    out_b = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention_mma_decode(qkv.cuda(), pages_b, table.cuda(), page, row_start, row_pos0, out_b,
                             rows, n, H, G, hd, scale, window, cos.cuda(), sin.cuda(), interleaved,
                             True, n_splits, scratch)
    assert torch.equal(out_b.cpu(), out_a.cpu())
    assert torch.equal(pages_b.cpu(), pages_a.cpu())
    # (that was with the splits merged inside the kernel by the last CTA to arrive; a merge
    # kernel after it gives the same bits, and so does a second launch on the same counters)
    for inside in (False, True):
        pages_d = pages.clone().cuda()
        out_d = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.attention_mma_decode(qkv.cuda(), pages_d, table.cuda(), page, row_start, row_pos0,
                                 out_d, rows, n, H, G, hd, scale, window, cos.cuda(), sin.cuda(),
                                 interleaved, True, n_splits, scratch, merge_inside=inside)
        assert torch.equal(out_d.cpu(), out_a.cpu())
    # a layer that reads another layer's cache: nothing is stored
    pages_c = pages_a.clone()
    out_c = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention_mma_decode(qkv.cuda(), pages_c, table.cuda(), page, row_start, row_pos0, out_c,
                             rows, n, H, G, hd, scale, window, cos.cuda(), sin.cuda(), interleaved,
                             False, n_splits, scratch)
    assert torch.equal(out_c.cpu(), out_a.cpu()) and torch.equal(pages_c.cpu(), pages_a.cpu())


@pytest.mark.parametrize("H, G, hd, page", [(8, 2, 64, 16), (32, 8, 128, 16), (8, 1, 128, 32),
                                           (4, 4, 64, 8), (2, 1, 128, 128), (4, 2, 256, 16),
                                           (2, 2, 192, 32)])
@pytest.mark.parametrize("two_tiles", [True, False])
def test_attention_tcgen05(ops, H, G, hd, page, two_tiles):
    """Prompt portions on the tcgen05 kernels (two query tiles per CTA, which head sizes up to
    128 use, and one): long rows (several key tiles, several query
    tiles), rows that start deep in a context, short rows; unused cache places hold NaN, as for
    the other attention kernels, and must not reach a result (rows that end in the middle of a
    page and of a key tile leave stale keys and values right behind their last position)."""
    ops.prepare([hd], verbose=False)
    if hd > 128 and two_tiles:
        pytest.skip("head sizes above 128 have the one-tile kernel only")
    rows = [(0, 300), (450, 40), (0, 17), (127, 2), (128, 129), (1000, 30), (60, 65), (0, 64)]
    global ATTN_ROWS
    saved = ATTN_ROWS
    ATTN_ROWS = rows
    ops.attention_tc_set_two_tiles(hd, two_tiles)
    try:
        case = attention_case("bfloat16", H, G, hd, page)
        pages = case["pages"]
        assert torch.isnan(pages.float()).any()
        q = case["wide"][:, :H * hd]
        out = torch.full((q.shape[0], H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        every = list(range(len(rows)))
        for _ in range(10):   # the warps of the kernel overlap differently from run to run
            out.fill_(float("nan"))
            ops.attention_tc(q, pages, case["table"], page, case["row_start"], case["row_pos0"],
                             out, None, len(rows), max(n for _, n in rows), H, G, hd,
                             1.0 / math.sqrt(hd))
            assert ops.attention_tc_error(hd) == 0
            check_attention(case, out.cpu().float(), every, "bfloat16", H, hd, None)
    finally:
        ATTN_ROWS = saved
        ops.attention_tc_set_two_tiles(hd, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_and_cache_write(ops, dtype, interleaved):
    H, G, hd, page, theta, max_pos = 3, 2, 48, 8, 50000.0, 300
    dt = DT[dtype]
    pos = torch.tensor([0, 1, 2, 250, 7, 8, 9, 10, 299], dtype=torch.int32)
    row = torch.tensor([0, 0, 0, 1, 2, 2, 2, 2, 3], dtype=torch.int32)
    n = len(pos)
    qkv = rand(n, (H + 2 * G) * hd, dtype=dt, seed=4)
    cos, sin = P.rope_tables(hd, max_pos, theta)
    table = torch.full((4, 38), -1, dtype=torch.int32)
    table[0, 0], table[1, 31], table[2, 0], table[2, 1], table[3, 37] = 5, 2, 9, 0, 7
    pages = torch.zeros(10, 2, G, page, hd, dtype=dt).cuda()
    buf = qkv.clone().cuda()
    ops.rope_kv_write(buf, pos.cuda(), row.cuda(), cos.cuda(), sin.cuda(), pages, table.cuda(),
                      page, H, G, hd, interleaved, True)
    q = qkv[:, :H * hd].float().view(n, H, hd).transpose(0, 1)
    k = qkv[:, H * hd:(H + G) * hd].float().view(n, G, hd).transpose(0, 1)
    v = qkv[:, (H + G) * hd:].float().view(n, G, hd)
    q_want = P.apply_rope(q, pos.long(), cos, sin, interleaved).transpose(0, 1).reshape(n, H * hd)
    k_want = P.apply_rope(k, pos.long(), cos, sin, interleaved).transpose(0, 1)
    got = buf.cpu().float()
    torch.testing.assert_close(got[:, :H * hd], q_want, **TOL[dtype])
    assert torch.equal(got[:, H * hd:], qkv[:, H * hd:].float())  # k, v of the buffer untouched
    pg = pages.cpu().float()
    for i in range(n):
        phys, off = int(table[row[i], pos[i] // page]), int(pos[i]) % page
        torch.testing.assert_close(pg[phys, 0, :, off], k_want[i], **TOL[dtype])
        assert torch.equal(pg[phys, 1, :, off], v[i])
    assert int((pg != 0).any(dim=-1).sum()) == n * 2 * G  # nothing else was written
    # write=False rotates q only
    pages2 = torch.zeros_like(pages)
    ops.rope_kv_write(qkv.clone().cuda(), pos.cuda(), row.cuda(), cos.cuda(), sin.cuda(), pages2,
                      table.cuda(), page, H, G, hd, interleaved, False)
    assert not pages2.any()


def test_sampling_greedy_ties_and_logprob(ops):
    V = 1000
    logits = rand(4, V, seed=5)
    logits[1, 700] = logits[1, 20] = 9.0   # a tie: the first maximum wins
    logits[2] = -1e30
    logits[2, 999] = 0.0
    out = torch.empty(4, dtype=torch.int32, device="cuda")
    lp = torch.empty(4, dtype=torch.float32, device="cuda")
    ops.sample(logits.cuda(), out, logprob_out=lp)
    want = logits.argmax(-1)
    want[1] = 20
    assert out.cpu().tolist() == want.tolist()
    torch.testing.assert_close(lp.cpu(), torch.log_softmax(logits, -1)[torch.arange(4), want],
                               rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n, V", [(1, 7), (5, 331), (8, 128256), (64, 50000)])
def test_argmax_many_blocks_per_row(ops, n, V):
    logits = rand(n, V, seed=3)
    logits[0, V - 1] = logits[0, V // 3] = 50.0      # a tie: the first maximum wins
    scratch = torch.zeros(ops.argmax_scratch_bytes(n), dtype=torch.uint8, device="cuda")
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    want = logits.argmax(-1)
    want[0] = V // 3
    for _ in range(3):   # the scratch resets itself
        out.fill_(-1)
        ops.argmax(logits.cuda(), out, scratch, n)
        assert out.cpu().tolist() == want.tolist()


@pytest.mark.parametrize("V", [8191, 8192, 8193, 70001])
def test_sampling_edges_of_the_cluster_kernel(ops, V):
    """Vocabularies around the size from which a cluster of CTAs serves a row (and one that no
    CTA's slice divides), many rows, a nucleus of almost nothing and of everything, a high and a
    low temperature, peaked rows, and the log-probability of the drawn token."""
    n = 150
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(n, V, generator=g) * 2.0
    logits[3] = -50.0
    logits[3, V - 1] = 10.0                    # all mass on the last token
    logits[4, : V // 2] += 30.0                # half the row far above the other half
    temps = torch.tensor([0.05, 0.3, 1.0, 1.0, 2.0, 5.0] * (n // 6))
    tops = torch.tensor([0.01, 0.5, 0.999, 1.0, 0.9, 0.2] * (n // 6))
    seed = torch.arange(n, dtype=torch.int64).cuda()
    ctr = torch.full((n,), 7, dtype=torch.int64).cuda()
    probs = torch.empty(n, V, dtype=torch.float32, device="cuda")
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    lp = torch.empty(n, dtype=torch.float32, device="cuda")
    ops.sample(logits.cuda(), out, temps.cuda(), tops.cuda(), seed, ctr, logprob_out=lp,
               probs_out=probs)
    got_all, tok = probs.cpu(), out.cpu().long()
    assert int(tok[3]) == V - 1
    want_lp = torch.log_softmax(logits, -1)[torch.arange(n), tok]
    torch.testing.assert_close(lp.cpu(), want_lp, rtol=1e-4, atol=1e-4)
    for r in range(0, n, 7):
        want = P.sampling_distribution(logits[r], float(temps[r]), float(tops[r]))
        got = got_all[r]
        differ = (got > 0) != (want > 0)
        assert differ.sum() <= 1, (r, int(differ.sum()))
        if not differ.any():
            torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-7)
        assert got[tok[r]] > 0 and abs(float(got.sum()) - 1.0) < 1e-4
    # a row's draw does not depend on its neighbours or on their number
    alone = torch.empty(1, dtype=torch.int32, device="cuda")
    for r in (0, 5, n - 1):
        ops.sample(logits[r:r + 1].cuda(), alone, temps[r:r + 1].cuda(), tops[r:r + 1].cuda(),
                   seed[r:r + 1], ctr[r:r + 1])
        assert int(alone) == int(tok[r])


@pytest.mark.parametrize("V", [331, 50000, 128256, 9001])
def test_sampling_distribution_and_draws(ops, V):
    logits = rand(3, V, seed=6, scale=2.0)
    temps = torch.tensor([0.7, 1.0, 1.3])
    tops = torch.tensor([0.9, 1.0, 0.5])
    probs = torch.empty(3, V, dtype=torch.float32, device="cuda")
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    seed = torch.tensor([1, 2, 3], dtype=torch.int64).cuda()
    ctr = torch.zeros(3, dtype=torch.int64).cuda()
    ops.sample(logits.cuda(), out, temps.cuda(), tops.cuda(), seed, ctr, probs_out=probs)
    for r in range(3):
        want = P.sampling_distribution(logits[r], float(temps[r]), float(tops[r]))
        got = probs[r].cpu()
        # the kept sets agree except possibly for tokens whose mass sits on the top-p edge
        differ = (got > 0) != (want > 0)
        assert differ.sum() <= 1
        if not differ.any():
            torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-7)
        assert got[out[r].item()] > 0
    # without a nucleus (no top_p given): the whole distribution at the row's temperature
    whole = torch.empty(3, V, dtype=torch.float32, device="cuda")
    ops.sample(logits.cuda(), out.clone(), temps.cuda(), None, seed, ctr, probs_out=whole)
    for r in range(3):
        torch.testing.assert_close(whole[r].cpu(), P.sampling_distribution(logits[r], float(temps[r]), 1.0),
                                   rtol=1e-4, atol=1e-7)
    # the same (seed, counter) draws the same token; counters walk through the distribution
    again = torch.empty(3, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), again, temps.cuda(), tops.cuda(), seed, ctr)
    assert torch.equal(out, again)
    n_draws = 4000
    big = logits[2:3].expand(n_draws, V).contiguous().cuda()
    draws = torch.empty(n_draws, dtype=torch.int32, device="cuda")
    ops.sample(big, draws, torch.full((n_draws,), 1.3).cuda(), torch.full((n_draws,), 0.5).cuda(),
               torch.full((n_draws,), 77, dtype=torch.int64).cuda(),
               torch.arange(n_draws, dtype=torch.int64).cuda())
    freq = torch.bincount(draws.cpu().long(), minlength=V).float() / n_draws
    want = P.sampling_distribution(logits[2], 1.3, 0.5)
    assert freq[want == 0].sum() <= 1.0 / n_draws * 2
    top = want.argsort(descending=True)[:5]
    torch.testing.assert_close(freq[top], want[top], rtol=0.3, atol=0.01)
