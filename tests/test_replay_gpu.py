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
           "C": [34, 95, 200, 61, 150, 333, 16, 640, 48, 100]}
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


def make_runner(model_dir, dtype, page_size, max_tokens, max_requests=4):
    from scratch_llm_b200.engine import ModelRunner, load_model
    model = load_model(model_dir, dtype, verbose=False)
    return ModelRunner(model, page_size, -(-max_tokens // page_size), max_requests)


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
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("way", ["whole", "tail", "portions", "mixed"])
def test_replay_matches_plain(way, name, dtype, model_dirs, expected):
    reqs, want = expected(name, dtype)
    steps = {"whole": T.whole, "tail": T.tail_one_by_one, "portions": T.changing_portions,
             "mixed": T.mixed}[way](reqs)
    peak = T.peak_tokens(steps)
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], peak)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    compare(got, want, dtype)
    assert not runner.cache.requests and all(
        g.pool.n_free == g.pool.n_pages for g in runner.cache.groups)
    if way == "mixed":
        # the pool is smaller than what all requests need together: pages were used again
        total_pages = sum(-(-len(t) // PAGE_SIZE[name]) for t in reqs.values())
        assert runner.cache.groups[0].pool.n_pages < total_pages


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


def test_long_prompt_takes_the_fused_tensor_core_path(tmp_path):
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
    assert 1000 >= linear.FUSED_GEMM_MIN_TOKENS
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
