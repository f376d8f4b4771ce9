"""Generation through the Python entry point on the GPU: greedy against the plain
implementation, long decoding, the first tokens of a sequence, sampling, a pool so small that
requests are set back."""

import pytest
import torch

from configs import CONFIGS, PAGE_SIZE
from plain import llama_plain as P

pytestmark = pytest.mark.gpu


def prompts_for(vocab, lengths, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def plain_weights(model_dir, dtype):
    cfg, w = P.read_model_dir(model_dir)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return cfg, w


def assert_greedy_consistent(cfg, w, prompt, generated, slack):
    """Every generated token is the plain model's argmax given the tokens before it, up to
    ``slack`` in the logit (0 would demand the exact argmax; rounding may swap near-ties)."""
    logits = P.forward(cfg, w, prompt + generated)
    for i, tok in enumerate(generated):
        row = logits[len(prompt) + i - 1]
        assert row[tok] >= row.max() - slack, (i, tok, int(row.argmax()), float(row.max() - row[tok]))


@pytest.mark.parametrize("dtype, slack", [("float32", 2e-5), ("bfloat16", 6e-2)])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain(name, dtype, slack, model_dirs):
    from scratch_llm_b200 import LLM, SamplingParams
    cfg, w = plain_weights(model_dirs[name], dtype)
    lengths = {"A": [5, 17, 33], "B": [1, 9, 40, 64, 100], "C": [15, 16, 17, 70]}[name]
    n_new = {"A": 16, "B": 24, "C": 20}[name]
    prompts = prompts_for(cfg["vocab_size"], lengths)
    llm = LLM(model_dirs[name], dtype=dtype, max_tokens=1024, page_size=PAGE_SIZE[name],
              max_batch_tokens=48, chunk_size=32)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new))
    assert [len(g) for g in got] == [n_new] * len(prompts)
    for p, g in zip(prompts, got):
        assert_greedy_consistent(cfg, w, p, g, slack)
    if dtype == "float32":
        assert got[0] == P.greedy(cfg, w, prompts[0], n_new)
    # the reference's name for a greedy batch gives the same
    from scratch_llm_b200 import batched_greedy_decode
    if dtype == "float32":
        assert batched_greedy_decode(llm, prompts, n_new) == got
    # one prompt alone gives what it gave in the batch
    alone = llm.generate(prompts[1], SamplingParams(temperature=0.0, max_tokens=n_new))
    if dtype == "float32":
        assert alone == got[1]
    else:
        assert_greedy_consistent(cfg, w, prompts[1], alone, slack)


@pytest.mark.parametrize("dtype, slack", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_long_decoding(dtype, slack, model_dirs):
    from scratch_llm_b200 import LLM, SamplingParams
    cfg, w = plain_weights(model_dirs["C"], dtype)
    prompt = prompts_for(331, [21])[0]
    llm = LLM(model_dirs["C"], dtype=dtype, max_tokens=640, page_size=16)
    got = llm.generate(prompt, SamplingParams(temperature=0.0, max_tokens=600))
    assert len(got) == 600
    assert_greedy_consistent(cfg, w, prompt, got, slack)


@pytest.mark.parametrize("dtype, tol", [("float32", dict(rtol=2e-5, atol=5e-6)),
                                        ("bfloat16", dict(rtol=3e-2, atol=3e-2))])
def test_first_tokens_of_a_sequence(dtype, tol, model_dirs):
    from scratch_llm_b200.engine import ModelRunner, RowInput, load_model
    cfg, w = plain_weights(model_dirs["B"], dtype)
    runner = ModelRunner(load_model(model_dirs["B"], dtype, verbose=False), 8, 16, 4)
    toks = [7, 300, 12]
    want = P.forward(cfg, w, toks)
    with torch.no_grad():
        runner.admit("x")
        first = runner.step([RowInput("x", toks[:1], [0])])
        second = runner.step([RowInput("x", toks[1:2], [0])])
        third = runner.step([RowInput("x", toks[2:], [0])])
    for got, pos in ((first, 0), (second, 1), (third, 2)):
        torch.testing.assert_close(got[0].cpu(), want[pos], **tol)


def test_small_pool_sets_requests_back_and_results_do_not_change(model_dirs):
    from scratch_llm_b200 import LLM, SamplingParams
    prompts = prompts_for(256, [30, 25, 28, 9, 33, 20])
    params = SamplingParams(temperature=0.0, max_tokens=40)
    big = LLM(model_dirs["A"], dtype="float32", max_tokens=2048, page_size=16)
    want = big.generate(prompts, params)
    small = LLM(model_dirs["A"], dtype="float32", max_tokens=160, page_size=16, max_requests=4)
    res = small.serve([__import__("scratch_llm_b200").Request(i, p, params)
                       for i, p in enumerate(prompts)])
    assert res.stats.preemptions > 0
    assert [list(c.token_ids) for c in res.completed] == want
    small.runner.cache.check()
    assert not small.runner.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(dtype, model_dirs):
    """With ``lookahead`` the next decode step is launched before the host has read the tokens
    of the one in flight (they reach the embedding on the device).  Tokens, log-probabilities,
    finish reasons and the cache's accounts are those of the plain loop: greedy and sampled,
    with stop tokens that end requests while a row of theirs is in flight, and with a pool so
    small that requests are set back."""
    from scratch_llm_b200 import LLM, Request, SamplingParams
    prompts = prompts_for(256, [30, 5, 28, 9, 17, 21])
    base = LLM(model_dirs["A"], dtype=dtype, max_tokens=2048, page_size=16, lookahead=False)
    greedy = base.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24))
    params = [SamplingParams(temperature=0.0, max_tokens=24, stop_ids=(greedy[0][3],)),
              SamplingParams(temperature=0.0, max_tokens=24, stop_ids=(greedy[1][10], greedy[1][0])),
              SamplingParams(temperature=0.8, top_p=0.9, max_tokens=19, seed=7),
              SamplingParams(temperature=0.0, max_tokens=1),
              SamplingParams(temperature=1.0, max_tokens=30, seed=8, stop_ids=(greedy[4][2],)),
              SamplingParams(temperature=0.0, max_tokens=2)]
    reqs = [Request(i, p, sp) for i, (p, sp) in enumerate(zip(prompts, params))]
    want = base.serve(reqs, want_logprobs=True)
    for kw in (dict(max_tokens=2048), dict(max_tokens=96, max_requests=4)):
        ahead = LLM(model_dirs["A"], dtype=dtype, page_size=16, lookahead=True, **kw)
        got = ahead.serve(reqs, want_logprobs=True)
        for a, b in zip(got.completed, want.completed):
            assert a.token_ids == b.token_ids and a.finish_reason == b.finish_reason
            assert a.logprobs == b.logprobs
        ahead.runner.cache.check()
        assert not ahead.runner.cache.requests
    assert any(c.finish_reason == "stop" for c in want.completed)
    # a pool so small that requests are set back while steps are launched ahead
    long = [Request(i, p, SamplingParams(temperature=0.0, max_tokens=40))
            for i, p in enumerate(prompts_for(256, [30, 25, 28, 9, 33, 20]))]
    want_long = base.serve(long)
    small = LLM(model_dirs["A"], dtype=dtype, max_tokens=160, page_size=16, max_requests=4,
                lookahead=True)
    got_long = small.serve(long)
    assert got_long.stats.preemptions > 0
    assert [c.token_ids for c in got_long.completed] == [c.token_ids for c in want_long.completed]
    small.runner.cache.check()
    assert not small.runner.cache.requests
    # step by step through submit()/step(): every token is reported once, by its own step
    llm = LLM(model_dirs["A"], dtype=dtype, max_tokens=2048, page_size=16, lookahead=True)
    for r in reqs:
        llm.submit(r)
    seen = {r.request_id: [] for r in reqs}
    while llm.has_work:
        for rid, tok in llm.step().items():
            seen[rid].append(tok)
    assert [tuple(seen[r.request_id]) for r in reqs] == [c.token_ids for c in want.completed]


def test_sampling_through_the_entry_point(model_dirs):
    from scratch_llm_b200 import LLM, SamplingParams
    llm = LLM(model_dirs["A"], dtype="float32", max_tokens=1024, page_size=16)
    prompts = prompts_for(256, [12, 7, 19])
    sp = [SamplingParams(temperature=0.9, top_p=0.95, max_tokens=12, seed=s) for s in (1, 2, 3)]
    batch = llm.generate(prompts, sp)
    # a request's draws depend on its own seed and count, not on the batch
    assert llm.generate(prompts[1], sp[1]) == batch[1]
    assert llm.generate(prompts[1], SamplingParams(temperature=0.9, top_p=0.95, max_tokens=12,
                                                   seed=99)) != batch[1]
    # stop ids end the generation and are kept
    greedy = llm.generate(prompts[0], SamplingParams(temperature=0.0, max_tokens=12))
    cut = llm.generate(prompts[0], SamplingParams(temperature=0.0, max_tokens=12,
                                                  stop_ids=(greedy[4],)))
    assert cut == greedy[:greedy.index(greedy[4]) + 1]
    # log-probabilities are those of the plain model
    cfg, w = plain_weights(model_dirs["A"], "float32")
    toks, lps = llm.generate_with_logprobs(prompts[2], SamplingParams(temperature=0.0, max_tokens=5))
    logits = P.forward(cfg, w, prompts[2] + toks)
    want = [float(torch.log_softmax(logits[len(prompts[2]) + i - 1], -1)[t])
            for i, t in enumerate(toks)]
    torch.testing.assert_close(torch.tensor(lps), torch.tensor(want), rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError, match="non-empty"):
        llm.generate([[]], SamplingParams(max_tokens=2))


def test_no_cpu_path():
    from scratch_llm_b200.kernels import ops
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.embed(torch.zeros(2, dtype=torch.int32), torch.zeros(4, 8), torch.zeros(2, 8))


@pytest.mark.parametrize("dtype, tol", [("float32", dict(rtol=2e-5, atol=5e-6)),
                                        ("bfloat16", dict(rtol=3e-2, atol=3e-2))])
def test_small_steps_padded_and_replayed_as_graphs(dtype, tol, model_dirs):
    """Steps of a few tokens (portions of prompts alone and beside decoded tokens) are padded
    to a few shapes and replayed as captured graphs.  Against a runner that launches every
    step plainly and unpadded: the same logits, graphs were replayed, and the cache holds the
    same keys and values (padding tokens store nothing)."""
    from scratch_llm_b200.engine import ModelRunner, RowInput, load_model
    model = load_model(model_dirs["B"], dtype, verbose=False)
    page = PAGE_SIZE["B"]
    runners = [ModelRunner(model, page, 64, 6, cuda_graphs=g) for g in (True, False)]
    assert runners[0].pad_small_steps and not runners[1].pad_small_steps
    runners[0].capture_padded_after = 2   # (shapes are captured later by default)
    vocab = CONFIGS["B"]["vocab_size"]
    g = torch.Generator().manual_seed(3)
    toks = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()  # noqa: E731
    for r in runners:
        for grp in r.cache.groups:
            grp.pages.zero_()    # the pools are compared whole below, and start as they came
        for rid in "abcd":
            assert r.admit(rid)
    # shapes repeat (19 and 21 tokens both pad to 32, ...), rows change places, some steps want
    # nothing, one row wants several places
    plan = [
        [("a", 19, [18])], [("b", 21, [20])], [("c", 30, [0, 29])], [("d", 17, [])],
        [("a", 1, [0]), ("b", 1, [0]), ("c", 5, [4])], [("c", 1, [0]), ("d", 7, [6]), ("a", 1, [0])],
        [("b", 3, [2]), ("a", 1, [0]), ("d", 1, [0])], [("d", 2, [0, 1]), ("c", 2, [1])],
        [("a", 40, []), ("b", 1, [0])], [("b", 33, []), ("c", 1, [0])], [("c", 37, [36]), ("d", 1, [0])],
        [("a", 2, [1]), ("b", 2, [1]), ("c", 2, [1]), ("d", 2, [1])],
        [("a", 3, [2]), ("b", 2, [1]), ("c", 4, [3]), ("d", 2, [1])],
    ]
    with torch.no_grad():
        for step in plan:
            rows = [RowInput(rid, toks(n), want) for rid, n, want in step]
            got = [r.step(rows) for r in runners]
            if got[1] is None:
                assert got[0] is None
                continue
            assert got[0].shape == got[1].shape
            torch.testing.assert_close(got[0].cpu(), got[1].cpu(), **tol)
    assert runners[0].replayed_steps >= 4 and runners[1].replayed_steps == 0
    # with every captured step dropped (as after a failed capture) capturing starts afresh
    runners[0]._captured.clear()
    before = runners[0].replayed_steps
    with torch.no_grad():
        for _ in range(3):
            rows = [RowInput(rid, toks(2), [1]) for rid in "abcd"]
            got = [r.step(rows) for r in runners]
            torch.testing.assert_close(got[0].cpu(), got[1].cpu(), **tol)
    assert runners[0].replayed_steps > before
    for a, b in zip((grp.pages for grp in runners[0].cache.groups),
                    (grp.pages for grp in runners[1].cache.groups)):
        if dtype == "float32":
            assert torch.equal(a.cpu(), b.cpu())
        else:
            torch.testing.assert_close(a.float().cpu(), b.float().cpu(), **tol)
    for r in runners:
        for rid in "abcd":
            r.release(rid)
        r.cache.check()


@pytest.mark.parametrize("dtype, slack", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_requests_arriving_while_others_decode(dtype, slack, model_dirs):
    """Requests arrive every other step, so that most steps mix a prompt (or a portion of one)
    with decoded tokens; the pool is small enough that requests are set back.  With padded
    steps captured at once and decode steps launched ahead, every token is what a runner
    without graphs and padding gives (32-bit: the same tokens; bfloat16: each token the plain
    model's choice up to rounding)."""
    import random
    from scratch_llm_b200 import LLM, Request, SamplingParams
    rng = random.Random(4)
    vocab = CONFIGS["B"]["vocab_size"]
    reqs = [Request(i, [rng.randrange(vocab) for _ in range(rng.randrange(2, 60))],
                    SamplingParams(temperature=0.0, max_tokens=rng.randrange(4, 28)))
            for i in range(36)]

    def run(graphs):
        llm = LLM(model_dirs["B"], dtype=dtype, max_tokens=176, page_size=PAGE_SIZE["B"],
                  max_requests=6, max_batch_tokens=48, chunk_size=32, lookahead=graphs)
        if graphs:
            assert llm.runner.pad_small_steps
            llm.runner.capture_padded_after = 2
        else:
            llm.runner.cuda_graphs = llm.runner.pad_small_steps = False
        out = {r.request_id: [] for r in reqs}
        nxt = step = 0
        while nxt < len(reqs) or llm.has_work:
            if nxt < len(reqs) and step % 2 == 0:
                llm.submit(reqs[nxt])
                nxt += 1
            if llm.has_work:
                for rid, tok in llm.step().items():
                    out[rid].append(tok)
            step += 1
        llm.runner.cache.check()
        assert not llm.runner.cache.requests
        return out, llm

    got, llm = run(True)
    assert llm.runner.replayed_steps > 20 and len(llm.runner._captured) > 3
    assert llm._sched.stats.preemptions > 0
    assert [len(got[r.request_id]) for r in reqs] == [r.params.max_tokens for r in reqs]
    if dtype == "float32":
        want, _ = run(False)
        assert got == want
    else:
        cfg, w = plain_weights(model_dirs["B"], dtype)
        for r in reqs[::3]:
            assert_greedy_consistent(cfg, w, list(r.prompt_ids), got[r.request_id], slack)


def test_serve_with_arrivals_on_a_test_clock(model_dirs):
    """``arrivals_s`` turns the request list into a stream (the reference's serve_continuous
    option): on a clock of the test's own, requests are queued when their time has come, the
    engine sleeps while nothing is live, every token has its time, and the tokens are those
    of the closed list."""
    from scratch_llm_b200 import LLM, Request, SamplingParams, serve_continuous
    prompts = prompts_for(256, [12, 30, 7, 21, 16])
    reqs = [Request(i, p, SamplingParams(temperature=0.0, max_tokens=6 + i))
            for i, p in enumerate(prompts)]
    llm = LLM(model_dirs["A"], dtype="float32", max_tokens=1024, page_size=16)
    want = llm.serve(reqs)
    now = [100.0]
    slept = []

    def clock():
        now[0] += 0.001           # every look at the clock costs a millisecond
        return now[0]

    def sleep(seconds):
        slept.append(seconds)
        now[0] += seconds

    arrivals = [0.0, 0.5, 0.5, 3.0, 0.2]
    got = serve_continuous(llm, reqs, arrivals_s=arrivals, clock=clock, sleep=sleep)
    assert [c.token_ids for c in got.completed] == [c.token_ids for c in want.completed]
    assert slept and all(s >= 0 for s in slept)     # request 3 comes after the others are done
    by_id = {c.request.request_id: c for c in got.completed}
    for i, c in by_id.items():
        assert len(c.token_times_s) == len(c.token_ids)
        assert list(c.token_times_s) == sorted(c.token_times_s)
        assert c.token_times_s[0] > c.start_s                  # no token before its arrival
        assert abs(c.start_s - (got.completed[0].start_s + arrivals[i])) < 1e-9
    # admission follows arrival: 0, then 4, then 1 and 2, then 3
    steps = [by_id[i].admitted_at_step for i in (0, 4, 1, 2, 3)]
    assert steps == sorted(steps) and steps[0] < steps[1] < steps[2] and steps[3] < steps[4]
    # the reference's comparator: waves of requests, the same tokens in more steps
    from scratch_llm_b200 import serve_static_wave
    small = LLM(model_dirs["A"], dtype="float32", max_tokens=1024, page_size=16, max_requests=2)
    waves = serve_static_wave(small, reqs)
    assert [c.token_ids for c in waves.completed] == [c.token_ids for c in want.completed]
    assert waves.stats.steps > small.serve(reqs).stats.steps
    with pytest.raises(ValueError, match="one offset per request"):
        llm.serve(reqs, arrivals_s=[0.0])
    with pytest.raises(ValueError, match=">= 0"):
        llm.serve(reqs, arrivals_s=[0.0, 1.0, -1.0, 0.0, 0.0])
    assert not llm.has_work


@pytest.mark.parametrize("dtype, slack", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_decode_steps_of_many_rows_are_padded_to_eights(dtype, slack, model_dirs):
    """More than 8 requests decode together and end one by one: their steps are padded to the
    next multiple of 8 rows, so that 13, 12, 11, ... rows replay one captured graph.  The
    tokens are those of a runner without graphs (32-bit: the same; bfloat16: each the plain
    model's choice up to rounding)."""
    from scratch_llm_b200 import LLM, Request, SamplingParams
    vocab = CONFIGS["C"]["vocab_size"]
    prompts = prompts_for(vocab, [9, 20, 3, 14, 7, 11, 5, 16, 8, 12, 6, 10, 4])
    reqs = [Request(i, p, SamplingParams(temperature=0.0, max_tokens=6 + 2 * i))
            for i, p in enumerate(prompts)]
    llm = LLM(model_dirs["C"], dtype=dtype, max_tokens=2048, page_size=PAGE_SIZE["C"],
              max_requests=16)
    got = llm.serve(reqs)
    decode_keys = [k for k in llm.runner._captured if isinstance(k[0], int)]
    assert {k[0] for k in decode_keys} <= {1, 2, 3, 4, 5, 6, 7, 8, 16}
    assert any(k[0] == 16 for k in decode_keys) and llm.runner.replayed_steps > 10
    if dtype == "float32":
        plain = LLM(model_dirs["C"], dtype=dtype, max_tokens=2048, page_size=PAGE_SIZE["C"],
                    max_requests=16, lookahead=False)
        plain.runner.cuda_graphs = plain.runner.pad_small_steps = False
        want = plain.serve(reqs)
        assert [c.token_ids for c in got.completed] == [c.token_ids for c in want.completed]
    else:
        cfg, w = plain_weights(model_dirs["C"], dtype)
        for r, c in list(zip(reqs, got.completed))[::3]:
            assert_greedy_consistent(cfg, w, list(r.prompt_ids), list(c.token_ids), slack)


def run_cli(args, stdin_text):
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root), PYTHONIOENCODING="utf-8")
    proc = subprocess.run([sys.executable, "-m", "scratch_llm_b200.chat_cli", *args],
                          input=stdin_text, capture_output=True, text=True, encoding="utf-8",
                          timeout=600, env=env, cwd=str(root))
    assert proc.returncode == 0, proc.stderr[-3000:]
    return proc.stdout


def test_command_line_with_token_ids(tmp_path):
    """``python -m scratch_llm_b200.chat_cli`` as a child process: it writes the model folder
    from a configuration (--random-weights), opens it, reads token ids from standard input and
    prints the greedy continuation, which is the plain model's."""
    import json
    (tmp_path / "cfg.json").write_text(json.dumps(CONFIGS["A"]))
    model = tmp_path / "model"
    prompts = prompts_for(CONFIGS["A"]["vocab_size"], [7, 19], seed=3)
    text = "".join(" ".join(map(str, p)) + "\n" for p in prompts)
    out = run_cli(["--model", str(model), "--random-weights", str(tmp_path / "cfg.json"),
                   "--seed", "4", "--max-tokens", "8", "--dtype", "float32"], text)
    cfg, w = P.read_model_dir(model)
    replies = [line.split("bot> ", 1)[1] for line in out.splitlines() if "bot> " in line]
    assert [[int(t) for t in r.split()] for r in replies] == \
        [P.greedy(cfg, w, p, 8) for p in prompts]


def test_command_line_with_a_tokenizer(tmp_path, model_dirs):
    """The same with a ``tokenizer.json`` in the reference's format beside the model: text in,
    chat template around it, greedy reply out until the end-of-turn token or --max-tokens."""
    import json
    import shutil
    from scratch_llm_b200.chat_cli import EOT, SPECIALS, render_for_completion, special_id
    from scratch_llm_b200.tokenizer import Tokenizer
    model = tmp_path / "model"
    shutil.copytree(model_dirs["C"], model)          # vocabulary 331 >= the tokenizer's 265 ids
    vocab = {str(i): bytes([i]).decode("latin-1") for i in range(256)}
    merges = [["t", "h"], ["th", "e"], [" ", "the"], ["i", "n"], [" ", "c"]]
    for k, (a, b) in enumerate(merges):
        vocab[str(256 + k)] = a + b
    for k, sp in enumerate(SPECIALS):
        vocab[str(261 + k)] = sp
    for i in range(265, CONFIGS["C"]["vocab_size"]):     # every id the model can produce has a text
        vocab[str(i)] = f"[{i}]"
    data = tmp_path / "data"
    data.mkdir()
    (data / "tokenizer.json").write_text(json.dumps(
        {"vocab": vocab, "merges": merges, "special_tokens": SPECIALS}))
    tok = Tokenizer.load(data / "tokenizer.json")
    out = run_cli(["--ckpt", str(model), "--data-dir", str(data), "--max-tokens", "6",
                   "--dtype", "float32"], "the cat in the hat\n")
    cfg, w = P.read_model_dir(model)
    eot = special_id(tok, EOT)
    specials = {special_id(tok, sp) for sp in SPECIALS}
    gen = P.greedy(cfg, w, render_for_completion([("user", "the cat in the hat")], tok), 6)
    if eot in gen:
        gen = gen[:gen.index(eot)]
    want = tok.decode([t for t in gen if t not in specials])
    assert f"bot> {want}\n" in out


def test_score_gives_the_log_probabilities_of_given_tokens(model_dirs):
    """``LLM.score`` (the reference's LocalBackend.score, src/scratch_llm/rollout/local.py:50-79):
    log-probabilities of given continuation tokens under the model, against the plain model's
    log-softmax; a long pair is cut into portions by the token budget."""
    from scratch_llm_b200 import LLM
    cfg, w = plain_weights(model_dirs["B"], "float32")
    llm = LLM(model_dirs["B"], dtype="float32", max_tokens=1024, page_size=8,
              max_batch_tokens=48)
    prompts = prompts_for(cfg["vocab_size"], [1, 9, 70], seed=8)
    conts = prompts_for(cfg["vocab_size"], [5, 1, 60], seed=9)
    got = llm.score(prompts, conts)
    for p, c, g in zip(prompts, conts, got):
        logp = torch.log_softmax(P.forward(cfg, w, p + c), dim=-1)
        want = [float(logp[len(p) - 1 + i, t]) for i, t in enumerate(c)]
        torch.testing.assert_close(torch.tensor(g), torch.tensor(want), rtol=1e-4, atol=1e-4)
    one = llm.score(prompts[1], conts[1])
    torch.testing.assert_close(torch.tensor(one), torch.tensor(got[1]), rtol=1e-5, atol=1e-5)
    dist = llm.distribution_logprobs(prompts[2], conts[2])
    p, c = prompts[2], conts[2]
    want = torch.log_softmax(P.forward(cfg, w, p + c), dim=-1)[len(p) - 1:len(p) - 1 + len(c)]
    assert dist.shape == (len(c), cfg["vocab_size"])
    torch.testing.assert_close(dist.cpu(), want, rtol=1e-4, atol=1e-4)
    assert not llm.runner.cache.requests
