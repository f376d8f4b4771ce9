"""Replay on the GPU: every way of cutting the same requests into steps gives the logits of
the plain implementation, in 32-bit and in bfloat16."""

import pytest
import torch

import trace_util as T
from configs import CONFIGS, PAGE_SIZE
from plain import llama_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 128, 64, 15, 16, 90, 31, 120],
           "B": [2, 9, 40, 64, 100, 130, 47, 17, 80, 33, 200, 8, 150],
           "C": [34, 95, 200, 61, 150, 333, 16, 640, 48, 100],
           "D": [2, 700, 130, 64, 450, 17, 333, 65, 600, 31, 129, 512]}
# D's shapes select the kernels of the full-size models; its mixed traces cut prompts into
# portions of up to 500 tokens, so that steps of more than 512 tokens with several long portions
# beside single tokens occur (launched as they are, not padded), the tcgen05 attention gets a
# row list of several entries and the fused tcgen05 gate/up product runs
MIXED = {"D": dict(sizes=(2, 3, 40, 130, 300, 500), prefill_part=0.9)}
# 32-bit: a few ulp of the largest logit per reduction; bfloat16: operands rounded to 8 bits
TOL = {"float32": dict(rtol=2e-5, atol=5e-6), "bfloat16": dict(rtol=3e-2, atol=3e-2)}


@pytest.fixture(scope="module")
def expected(model_dirs):
    """Plain logits [S, V] per configuration, dtype and request.  For bfloat16 the plain model
    runs in 32-bit on the weights rounded to bfloat16, which is what the engine holds."""
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cfg, w = P.read_model_dir(model_dirs[name])
            if dtype == "bfloat16":
                w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
            reqs = T.make_requests(cfg["vocab_size"], LENGTHS[name], seed=11)
            cache[(name, dtype)] = (reqs, {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()})
        return cache[(name, dtype)]
    return get


def make_runner(model_dir, dtype, page_size, max_tokens, max_requests=4, **kw):
    from scratch_llm_b200.engine import ModelRunner, load_model
    model = load_model(model_dir, dtype, verbose=False)
    return ModelRunner(model, page_size, -(-max_tokens // page_size), max_requests, **kw)


def ways(name):
    mixed = (lambda r: T.mixed(r, **MIXED[name])) if name in MIXED else T.mixed
    return {"whole": T.whole, "tail": T.tail_one_by_one, "portions": T.changing_portions,
            "mixed": mixed}


def compare(got, want_logits, dtype):
    assert got, "the trace produced no logits"
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        ref = want_logits[rid][pos]
        worst = max(worst, float((row - ref).abs().max()))
        torch.testing.assert_close(row, ref, **TOL[dtype],
                                   msg=lambda m: f"request {rid} position {pos}: {m}")
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, page", [("A", 16), ("B", 8), ("C", 16), ("D", 16), ("D", 64)])
@pytest.mark.parametrize("way", ["whole", "tail", "portions", "mixed"])
def test_replay_matches_plain(way, name, page, dtype, model_dirs, expected, monkeypatch):
    """Free pages hold NaN (the pool at the start, and every page that is given back): a
    kernel that lets a place beyond a request's context reach a result fails here."""
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.parts import linear
    if name == "D":
        # the fused tcgen05 gate/up product would wait for 1,024 tokens at D's short reduction
        # (a choice of speed): here it runs from 448 on, as it does at the full-size widths
        monkeypatch.setattr(linear, "FUSED_GEMM_ALWAYS", linear.FUSED_GEMM_MIN_TOKENS)
    reqs, want = expected(name, dtype)
    steps = ways(name)[way](reqs)
    peak = T.peak_tokens(steps, round_to=max(64, page))
    runner = make_runner(model_dirs[name], dtype, page, peak, poison_free_pages=True)
    before = dict(ops.launch_counts)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    ops.check_kernel_errors()
    assert len(got) == sum(len(t) for t in reqs.values())
    compare(got, want, dtype)
    assert not runner.cache.requests and all(
        g.pool.n_free == g.pool.n_pages for g in runner.cache.groups)
    if way == "mixed":
        # the pool is smaller than what all requests need together: pages were used again
        total_pages = sum(-(-len(t) // page) for t in reqs.values())
        assert runner.cache.groups[0].pool.n_pages < total_pages
    if way == "mixed" and name == "D":
        ran = {k: v - before.get(k, 0) for k, v in ops.launch_counts.items()}
        if dtype == "bfloat16":
            # the kernels that the full-size models spend their time in all ran in this trace
            # (gemv_tma_sink: decode steps in which a product fed the residual stream itself
            # and the norm after it was finished by the next product)
            for op in ("gemv_tma", "gemv_tma_sink", "attention_mma_decode", "attention_tc",
                       "gemm_tc"):
                assert ran.get(op, 0) > 0, f"{op} never ran: {ran}"


def is_large_mixed(step):
    """More than 512 tokens (launched as it is, not padded), at least two portions that fill a
    128-query tile of the tcgen05 attention (32 tokens x 4 heads of a group), a single token."""
    sizes = [len(e["tokens"]) for e in step["entries"]]
    return sum(sizes) > 512 and sum(n >= 32 for n in sizes) >= 2 and 1 in sizes


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_mixed_steps(dtype, model_dirs, monkeypatch):
    """Steps of several hundred tokens that hold two or three long prompt portions beside
    decoded tokens of other requests, as a scheduler with a large token budget builds them all
    the time; pages are used again and free pages hold NaN."""
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.parts import linear
    monkeypatch.setattr(linear, "FUSED_GEMM_ALWAYS", linear.FUSED_GEMM_MIN_TOKENS)
    cfg, w = P.read_model_dir(model_dirs["D"])
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    lengths = [700, 450, 130, 600, 512, 333, 650, 280, 520, 64, 400]
    reqs = T.make_requests(cfg["vocab_size"], lengths, seed=31)
    want = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
    steps = T.large_mixed(reqs)
    assert sum(is_large_mixed(s) for s in steps) >= 2
    peak = T.peak_tokens(steps)
    assert peak < sum(-(-n // 64) * 64 for n in lengths) // 2
    runner = make_runner(model_dirs["D"], dtype, 16, peak, poison_free_pages=True)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    ops.check_kernel_errors()
    assert len(got) == sum(lengths)
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [1, 2, 4, 7, 8, 16, 32, 128])
def test_chunk_sizes_and_lengths_around_them(chunk, dtype, model_dirs):
    """Prompts of C-1, C, C+1 and 3C+1 tokens (plus three decoded ones) fed in chunks of C, for
    the chunk sizes of the reference's sweep (tests/test_chunked_prefill.py:99-140 there): one
    chunk, exactly one chunk, two chunks, a ragged last chunk."""
    cfg, w = P.read_model_dir(model_dirs["D"])
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    lengths = [n + 3 for n in (chunk - 1, chunk, chunk + 1, 3 * chunk + 1) if n >= 1]
    reqs = T.make_requests(cfg["vocab_size"], lengths, seed=100 + chunk)
    want = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
    steps = T.chunks_of(reqs, chunk)
    runner = make_runner(model_dirs["D"], dtype, 16, T.peak_tokens(steps), poison_free_pages=True)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    assert len(got) == sum(lengths)
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, model_dirs, expected, tmp_path):
    reqs, want = expected("B", dtype)
    steps = T.mixed(reqs, seed=3)
    # some steps want nothing, some only a few places
    for s in steps[::3]:
        for e in s["entries"]:
            e["want"] = []
    for s in steps[1::3]:
        for e in s["entries"]:
            e["want"] = e["want"][-1:]
    got = T.run_program(model_dirs["B"], dtype, steps, tmp_path / "out", T.peak_tokens(steps),
                        CONFIGS["B"]["vocab_size"], extra=["--page-size", "8"])
    compare(got, want, dtype)


def test_cutting_does_not_change_logits_beyond_rounding(model_dirs, expected):
    reqs, _ = expected("C", "float32")
    runner = make_runner(model_dirs["C"], "float32", 16, T.peak_tokens(T.whole(reqs)))
    with torch.no_grad():
        a = T.run_in_process(runner, T.whole(reqs))
        b = T.run_in_process(runner, T.changing_portions(reqs))
        c = T.run_in_process(runner, T.tail_one_by_one(reqs))
    for key in a:
        torch.testing.assert_close(a[key], b[key], rtol=1e-5, atol=2e-6)
        torch.testing.assert_close(a[key], c[key], rtol=1e-5, atol=2e-6)


#: bfloat16, the four cuttings against each other, as a fraction of the row's largest logit.
#: The cuttings share every rounding point (norm output, q and k after the rotation, the cache,
#: probabilities, attention output, activation, product outputs) but not their kernels, so they
#: differ by a few bfloat16 roundings that fall the other way, never by a key that one of them
#: masks and another does not (which moves a row by tens of percent).  Worst seen: 0.0066 (C)
#: and 0.0106 (D) of the row's largest logit; the bounds are about twice that.
BF16_CUTTING_BOUND = {"C": 0.015, "D": 0.02}


@pytest.mark.parametrize("name", ["C", "D"])
def test_cutting_does_not_change_bfloat16_logits_beyond_rounding(name, model_dirs, expected):
    """The four ways of cutting against EACH OTHER in bfloat16, and their greedy tokens equal
    wherever the plain model's margin between its two best tokens exceeds the bound."""
    reqs, want = expected(name, "bfloat16")
    page = PAGE_SIZE[name]
    results = {}
    for way, make in ways(name).items():
        steps = make(reqs)
        runner = make_runner(model_dirs[name], "bfloat16", page,
                             T.peak_tokens(steps, round_to=max(64, page)))
        with torch.no_grad():
            results[way] = T.run_in_process(runner, steps)
    base = results["whole"]
    worst = 0.0
    for way, got in results.items():
        assert got.keys() == base.keys()
        for key, row in got.items():
            top = float(base[key].abs().max())
            worst = max(worst, float((row - base[key]).abs().max()) / top)
    print(f"config {name}: worst difference between two cuttings = {worst:.4f} of the row maximum")
    assert worst <= BF16_CUTTING_BOUND[name]
    for key, ref_row in base.items():
        ref = want[key[0]][key[1]]
        best2 = torch.topk(ref, 2).values
        if float(best2[0] - best2[1]) > 2 * BF16_CUTTING_BOUND[name] * float(ref.abs().max()):
            tokens = {int(results[way][key].argmax()) for way in results}
            assert tokens == {int(ref.argmax())}, f"{key}: greedy tokens {tokens}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_hand_over_where_only_some_products_can(dtype, tmp_path):
    """A feed-forward width that the persistent small-batch product does not take (1,000 is no
    multiple of 512): in decode steps the output projection still feeds the residual stream
    itself and gate/up finishes the norm, while the down projection returns its output as
    usual and the next layer's norm runs as a kernel.  Logits match the plain model."""
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.weights import write_random_model
    raw = {**CONFIGS["D"], "intermediate_size": 1000, "num_hidden_layers": 3}
    d = write_random_model(config_from_dict(raw), tmp_path / "odd_ff", 6)
    cfg, w = P.read_model_dir(d)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    reqs = T.make_requests(cfg["vocab_size"], [40, 3, 70], seed=9)
    want = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
    steps = T.mixed(reqs, seed=2)
    runner = make_runner(d, dtype, 16, T.peak_tokens(steps), poison_free_pages=True)
    before = dict(ops.launch_counts)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    compare(got, want, dtype)
    sinks = ops.launch_counts.get("gemv_tma_sink", 0) - before.get("gemv_tma_sink", 0)
    assert (sinks > 0) == (dtype == "bfloat16")


def test_long_prompt_takes_the_fused_tensor_core_path(tmp_path, monkeypatch):
    """A prompt of 1,000 tokens in one step runs gate/up + SwiGLU on the tcgen05 kernel
    (shorter ones use other kernels); its logits still match the plain implementation."""
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.parts import linear
    from scratch_llm_b200.weights import write_random_model
    raw = {**CONFIGS["C"], "max_position_embeddings": 1100}
    d = write_random_model(config_from_dict(raw), tmp_path / "long", 5)
    cfg, w = P.read_model_dir(d)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    reqs = T.make_requests(cfg["vocab_size"], [1000], seed=4)
    monkeypatch.setattr(linear, "FUSED_GEMM_ALWAYS", linear.FUSED_GEMM_MIN_TOKENS)
    assert 1000 >= linear.FUSED_GEMM_ALWAYS
    want = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
    steps = T.whole(reqs)
    for s in steps:   # logits at a few places only: the first, one in the middle, the last 40
        s["entries"][0]["want"] = [0, 500] + list(range(960, 1000))
    runner = make_runner(d, "bfloat16", 16, 1024, max_requests=1)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    assert ops.gemm_tc_error() == 0
    compare(got, want, "bfloat16")


@pytest.fixture(scope="module")
def llama8b_layers(tmp_path_factory):
    """Two layers at Llama-3-8B layer sizes (width 4096, 32 heads over 8 kv heads of size 128,
    feed-forward 14336) with a smaller vocabulary that is no power of two; weights stored in
    bfloat16, so both precisions start from the same values."""
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.weights import write_random_model
    raw = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=2,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=14336, vocab_size=16001, rope_theta=500000.0, rms_norm_eps=1e-5,
               tie_word_embeddings=False, max_position_embeddings=2048, torch_dtype="bfloat16")
    d = write_random_model(config_from_dict(raw), tmp_path_factory.mktemp("llama8b_layers"), 8)
    cfg, w = P.read_model_dir(d)
    reqs = T.make_requests(cfg["vocab_size"], [900, 70], seed=21)
    want = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
    return d, reqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llama8b_layer_sizes(dtype, llama8b_layers):
    """The kernels at the sizes they are tuned for: the long request's prompt runs through the
    tcgen05 attention and the fused tcgen05 gate/up product (bfloat16), its last tokens and the
    short request through the decode kernels, mixed in one batch."""
    from scratch_llm_b200.kernels import ops
    d, reqs, want = llama8b_layers
    long_id, short_id = list(reqs)
    a, b = reqs[long_id], reqs[short_id]
    steps = [
        {"step": 0, "entries": [{"id": long_id, "tokens": a[:850], "want": [0, 400, 849]}], "end": []},
        {"step": 1, "entries": [{"id": long_id, "tokens": a[850:880], "want": list(range(30))},
                                {"id": short_id, "tokens": b[:40], "want": [39]}], "end": []}]
    for i in range(20):   # both requests decode side by side
        steps.append({"step": 2 + i, "entries": [
            {"id": long_id, "tokens": a[880 + i:881 + i], "want": [0]},
            {"id": short_id, "tokens": b[40 + i:41 + i], "want": [0]}], "end": []})
    steps.append({"step": 22, "entries": [{"id": short_id, "tokens": b[60:], "want": list(range(10))}],
                  "end": [long_id, short_id]})
    runner = make_runner(d, dtype, 16, 1024, max_requests=2)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    assert ops.gemm_tc_error() == 0 and ops.attention_tc_error(128) == 0
    # 32-bit: at these reduction lengths (4096 and 14336) the plain implementation itself moves
    # by 1.5e-5 between one and eight CPU threads and is 1.1e-5 away from its float64 run, on
    # logits up to 6.4; the bound leaves room for both sides' rounding and no more
    # bfloat16: with reductions over 4096 and 14336 rounded operands every path of the engine
    # (tensor-core prefill, library product, streaming decode kernels, token by token) lands
    # 1.2-2.0 % of the row's largest logit away from the plain 32-bit model, the same positions
    # being worst on every path: that is the precision of the format at this width.  The bound
    # is twice the worst seen.
    for (rid, pos), row in sorted(got.items()):
        ref = want[rid][pos]
        tol = dict(rtol=2e-4, atol=6e-5) if dtype == "float32" else \
            dict(rtol=3e-2, atol=0.04 * float(ref.abs().max()))
        torch.testing.assert_close(row, ref, **tol,
                                   msg=lambda m: f"request {rid} position {pos}: {m}")
