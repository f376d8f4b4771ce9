"""The scheduler's decisions, without a GPU: a stand-in step function whose next token is a
function of the sequence so far."""

import random
import zlib

import pytest

from scratch_llm_b200.cache import CacheManager
from scratch_llm_b200.engine.scheduler import Request, Scheduler, SchedulerStats
from scratch_llm_b200.parts import KVSpec
from scratch_llm_b200.sampling import SamplingParams

VOCAB = 97


def next_token(tokens):
    return zlib.crc32(repr(list(tokens)).encode()) % VOCAB


def oracle(prompt, params, max_position=10_000):
    toks, out = list(prompt), []
    while True:
        t = next_token(toks)
        toks.append(t)
        out.append(t)
        if t in params.stop_ids or len(out) >= params.max_tokens or len(toks) >= max_position:
            return out


def make(n_pages, page_size=4, max_requests=4, max_position=256, **kw):
    cache = CacheManager([KVSpec(1, 16, None)], [None], page_size, n_pages, max_requests)
    return Scheduler(cache, max_position, vocab_size=VOCAB, **kw), cache


def run(sched, cache, log=None, limit=10_000):
    for _ in range(limit):
        if not sched.has_work:
            break
        rows = sched.plan()
        assert rows, "a step with nothing in it"
        assert sum(r.n for r in rows) <= sched.max_batch_tokens
        assert len({id(r.seq) for r in rows}) == len(rows)
        for r in rows:
            assert r.start == cache.requests[r.seq.request.request_id].n_tokens
            assert 1 <= r.n <= len(r.seq.tokens) - r.start
            assert r.samples == (r.start + r.n == len(r.seq.tokens))
        sched.commit_rows(rows)
        sampled = [next_token(r.seq.tokens) for r in rows if r.samples]
        if log is not None:
            log.append([(r.seq.request.request_id, r.start, r.n, r.samples) for r in rows])
        sched.complete(rows, sampled)
        cache.check()
    else:
        raise AssertionError("the scheduler did not finish")
    assert not cache.requests
    assert cache.free_pages() == [g.pool.n_pages for g in cache.groups]


def greedy(n):
    return SamplingParams(temperature=0.0, max_tokens=n)


def test_mixed_steps_budget_and_portions():
    sched, cache = make(n_pages=200, max_batch_tokens=16, chunk_size=10)
    reqs = [Request("a", list(range(5)), greedy(6)), Request("b", list(range(23)), greedy(3)),
            Request("c", list(range(40, 52)), greedy(2))]
    for r in reqs:
        sched.submit(r)
    log = []
    run(sched, cache, log)
    # step 0: a whole (5), b's first portion (10, the chunk cap), c gets the last 1 of the budget
    assert log[0] == [("a", 0, 5, True), ("b", 0, 10, False), ("c", 0, 1, False)]
    # step 1: a decodes beside portions of b and c: one batch
    assert log[1][0] == ("a", 5, 1, True)
    assert ("b", 10, 10, False) in log[1] and ("c", 1, 5, False) in log[1]
    for r in reqs:
        assert sched.finished[r.request_id].generated == oracle(r.prompt_ids, r.params)
    assert sched.stats.preemptions == 0
    assert sched.stats.prefill_tokens == 5 + 23 + 12
    assert sched.stats.decode_tokens == (6 - 1) + (3 - 1) + (2 - 1)


def test_stats_of_the_held_pages():
    """What the held pages waste: sampled while requests are live, between 0 and the share a
    request's last page can leave empty."""
    sched, cache = make(n_pages=200, page_size=4, max_requests=4, max_batch_tokens=64)
    for i in range(6):
        sched.submit(Request(i, [1] * (3 + 2 * i), greedy(20)))
    run(sched, cache)
    st = sched.stats
    assert st.waste_samples and all(0.0 <= w < 0.75 for w in st.waste_samples)
    assert st.waste_mean is not None and 0.0 < st.waste_mean < 0.5
    assert 4 <= st.allocated_peak_tokens <= 4 * (13 + 20 + 4)
    assert SchedulerStats().waste_mean is None


def test_first_come_first_served_and_slots():
    sched, cache = make(n_pages=200, max_requests=2, max_batch_tokens=64)
    for i in range(5):
        sched.submit(Request(i, [i + 1] * 3, greedy(2 + i)))
    log = []
    run(sched, cache, log)
    first_seen = {}
    for s, rows in enumerate(log):
        assert len(rows) <= 2
        for rid, *_ in rows:
            first_seen.setdefault(rid, s)
    assert [first_seen[i] for i in range(5)] == sorted(first_seen[i] for i in range(5))
    assert all(sched.finished[i].generated == oracle([i + 1] * 3, greedy(2 + i)) for i in range(5))


def test_finish_reasons():
    sched, cache = make(n_pages=200, max_position=12)
    p_stop = SamplingParams(temperature=0.0, max_tokens=50, stop_ids=())
    first = oracle([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=4))
    with_stop = SamplingParams(temperature=0.0, max_tokens=9, stop_ids=(first[2],))
    sched.submit(Request("one", [1, 2, 3], greedy(1)))       # finishes with its first token
    sched.submit(Request("stop", [1, 2, 3], with_stop))
    sched.submit(Request("edge", [7] * 6, SamplingParams(temperature=0.0, max_tokens=6)))
    run(sched, cache)
    assert sched.finished["one"].generated == first[:1]
    assert sched.finished["one"].finish_reason == "length"
    stop_at = first.index(first[2])
    assert sched.finished["stop"].generated == first[:stop_at + 1]  # the stop token is kept
    assert sched.finished["stop"].finish_reason == "stop"
    assert len(sched.finished["edge"].tokens) == 12
    assert sched.finished["edge"].finish_reason in ("length", "max_position")
    with pytest.raises(ValueError, match="exceeds max_position"):
        sched.submit(Request("long", [1] * 6, p_stop))


def test_submit_errors():
    sched, _ = make(n_pages=4, page_size=4)
    with pytest.raises(ValueError, match="non-empty"):
        sched.submit(Request("e", [], greedy(1)))
    with pytest.raises(ValueError, match="out of range"):
        sched.submit(Request("v", [VOCAB], greedy(1)))
    with pytest.raises(ValueError, match="could never finish"):
        sched.submit(Request("big", [1] * 10, greedy(8)))   # 17 places > 16
    sched.submit(Request("ok", [1] * 10, greedy(7)))
    with pytest.raises(ValueError, match="already submitted"):
        sched.submit(Request("ok", [1], greedy(1)))


def test_pages_run_out_the_newest_request_is_set_back():
    # 8 pages of 4: two requests of 8 + 9 tokens fit at first, not to their ends
    sched, cache = make(n_pages=8, page_size=4, max_batch_tokens=64)
    reqs = [Request("old", [3] * 8, greedy(12)), Request("new", [5] * 9, greedy(12))]
    for r in reqs:
        sched.submit(r)
    log = []
    run(sched, cache, log)
    assert sched.stats.preemptions >= 1
    assert sched.finished["old"].n_preempted == 0     # the older request is never the victim
    assert sched.finished["new"].n_preempted >= 1
    for r in reqs:
        assert sched.finished[r.request_id].generated == oracle(r.prompt_ids, r.params)
    # after it was set back, "new" came in again with its prompt and its generated tokens
    again = [row for rows in log for row in rows if row[0] == "new" and row[1] == 0]
    assert len(again) >= 2 and again[-1][2] > 9


def test_reserve_full_never_sets_back_and_serialises():
    sched, cache = make(n_pages=8, page_size=4, max_batch_tokens=64, admission="reserve_full")
    reqs = [Request("a", [3] * 8, greedy(12)), Request("b", [5] * 9, greedy(12)),
            Request("c", [6] * 2, greedy(3))]
    for r in reqs:
        sched.submit(r)
    log = []
    run(sched, cache, log)
    assert sched.stats.preemptions == 0
    live = [{rid for rid, *_ in rows} for rows in log]
    assert not any({"a", "b"} <= s for s in live)       # 5 + 5 pages do not fit 8 together
    assert not any("c" in s and "b" not in s for s in live[:-4])  # no skipping ahead of b
    for r in reqs:
        assert sched.finished[r.request_id].generated == oracle(r.prompt_ids, r.params)


def test_prompt_portion_is_cut_to_the_pages_that_are_free():
    sched, cache = make(n_pages=6, page_size=4, max_batch_tokens=64)
    sched.submit(Request("a", [1] * 13, greedy(2)))   # 4 pages
    sched.submit(Request("b", [2] * 15, greedy(2)))   # wants 4, 2 are free
    log = []
    run(sched, cache, log)
    assert log[0] == [("a", 0, 13, True), ("b", 0, 8, False)]
    for rid, p in (("a", [1] * 13), ("b", [2] * 15)):
        assert sched.finished[rid].generated == oracle(p, greedy(2))


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_small_pool(seed):
    rng = random.Random(seed)
    sched, cache = make(n_pages=rng.choice([12, 20, 40]), page_size=rng.choice([2, 4, 8]),
                        max_requests=rng.choice([2, 3, 5]),
                        max_batch_tokens=rng.choice([8, 24, 100]),
                        chunk_size=rng.choice([None, 3, 16]), max_position=80)
    reqs = []
    pool_tokens = cache.groups[0].pool.n_pages * cache.page_size
    for i in range(14):
        n_p, n_g = rng.randint(1, 30), rng.randint(1, 20)
        if n_p + n_g - 1 > pool_tokens or n_p + n_g > 80:
            continue
        stop = (rng.randrange(VOCAB),) if rng.random() < 0.3 else ()
        reqs.append(Request(i, [rng.randrange(VOCAB) for _ in range(n_p)],
                            SamplingParams(temperature=0.0, max_tokens=n_g, stop_ids=stop)))
        sched.submit(reqs[-1])
    run(sched, cache)
    for r in reqs:
        assert sched.finished[r.request_id].generated == oracle(r.prompt_ids, r.params, 80)
    assert sched.stats.steps == len(sched.stats.tokens_per_step)


def run_ahead(sched, cache, limit=10_000):
    """The loop of the entry point with a step planned ahead: the next step is planned (and its
    rows committed) before the tokens of the step in flight are known."""
    in_flight, n_ahead = None, 0
    for _ in range(limit):
        if not sched.has_work:
            break
        cur = in_flight
        if cur is None:
            cur = sched.plan()
            assert cur
            sched.commit_rows(cur)
        in_flight = None
        # the tokens of `cur`: each from the tokens its request had when the row ran (rows planned
        # ahead ran with the pending token in place, which complete() has appended by now)
        alive_before = [not r.seq.finish_reason for r in cur]
        ahead = sched.plan_ahead(cur)
        if ahead is not None:
            rows = [r for r, _ in ahead]
            sampling = [r.seq for r in cur if r.samples]
            for r, j in ahead:
                assert sampling[j] is r.seq and r.n == 1 and r.samples
                assert r.start == cache.requests[r.seq.request.request_id].n_tokens == len(r.seq.tokens)
            sched.commit_rows(rows)
            in_flight = rows
            n_ahead += 1
        sampled = [next_token(r.seq.tokens) if a else -1
                   for r, a in zip(cur, alive_before) if r.samples]
        sched.complete(cur, sampled)
        cache.check()
    else:
        raise AssertionError("the scheduler did not finish")
    assert not cache.requests
    assert cache.free_pages() == [g.pool.n_pages for g in cache.groups]
    return n_ahead


@pytest.mark.parametrize("seed", range(6))
def test_steps_planned_ahead_give_the_same_tokens(seed):
    rng = random.Random(100 + seed)
    sched, cache = make(n_pages=rng.choice([30, 60, 200]), page_size=rng.choice([2, 4, 8]),
                        max_requests=rng.choice([2, 3, 5]),
                        max_batch_tokens=rng.choice([8, 24, 100]),
                        chunk_size=rng.choice([None, 3, 16]), max_position=80)
    reqs = []
    pool_tokens = cache.groups[0].pool.n_pages * cache.page_size
    for i in range(12):
        n_p, n_g = rng.randint(1, 30), rng.randint(1, 20)
        if n_p + n_g - 1 > pool_tokens or n_p + n_g > 80:
            continue
        stop = (rng.randrange(VOCAB),) if rng.random() < 0.5 else ()
        reqs.append(Request(i, [rng.randrange(VOCAB) for _ in range(n_p)],
                            SamplingParams(temperature=0.0, max_tokens=n_g, stop_ids=stop)))
        sched.submit(reqs[-1])
    n_ahead = run_ahead(sched, cache)
    for r in reqs:
        assert sched.finished[r.request_id].generated == oracle(r.prompt_ids, r.params, 80)
    assert n_ahead > 0


def test_plan_ahead_decisions():
    sched, cache = make(n_pages=50, max_batch_tokens=64)
    sched.submit(Request("a", [1, 2, 3], greedy(3)))
    sched.submit(Request("b", [4, 5], SamplingParams(temperature=0.0, max_tokens=8, stop_ids=(7,))))
    rows = sched.plan()
    sched.commit_rows(rows)
    ahead = sched.plan_ahead(rows)
    # both requests decode their pending token next; places follow the order of the sampling rows
    assert [(r.seq.request.request_id, r.start, r.n, j) for r, j in ahead] == [("a", 3, 1, 0),
                                                                               ("b", 2, 1, 1)]
    sched.commit_rows([r for r, _ in ahead])
    sched.complete(rows, [9, 7])          # b's pending token was its stop token
    assert "b" in sched.finished and sched.finished["b"].generated == [7]
    rows2 = [r for r, _ in ahead]
    # a's second token ends it for certain (max_tokens = 3 would be reached by the third), so
    # the step after rows2 still holds a; then nothing is left to plan ahead
    ahead2 = sched.plan_ahead(rows2)
    assert [(r.seq.request.request_id, j) for r, j in ahead2] == [("a", 0)]
    sched.commit_rows([r for r, _ in ahead2])
    sched.complete(rows2, [11, 12])       # b's row is dropped: it had ended
    assert sched.finished["b"].generated == [7]
    assert sched.plan_ahead([r for r, _ in ahead2]) is None   # a's pending token is its last
    sched.complete([r for r, _ in ahead2], [13])
    assert sched.finished["a"].generated == [9, 11, 13] and not sched.has_work
    # a queued request, or a prompt that is half read, sends the decision back to plan()
    sched2, cache2 = make(n_pages=50, max_batch_tokens=4, max_requests=1)
    sched2.submit(Request("x", [1, 2, 3], greedy(4)))
    sched2.submit(Request("y", [1], greedy(2)))
    rows = sched2.plan()
    sched2.commit_rows(rows)
    assert sched2.plan_ahead(rows) is None


def test_padding_plan_of_small_steps():
    """Steps of many shapes fall on few padded shapes; nothing wanted stays nothing wanted."""
    from scratch_llm_b200.engine.batch import PAD_MAX_TOKENS, pad_plan
    seen = set()
    for n_tokens in range(1, PAD_MAX_TOKENS + 1):
        for n_single, n_multi, n_out in ((0, 1, 1), (3, 1, 4), (9, 2, 0), (0, 3, n_tokens)):
            if n_single + 2 * n_multi > n_tokens:
                continue
            plan = pad_plan(n_tokens, n_single, n_multi, n_out)
            assert n_tokens <= plan.n_tokens < n_tokens + (16 if n_tokens <= 128 else 64)
            assert n_single <= plan.n_single < n_single + 8 and plan.n_single % 8 == 0
            assert n_multi <= plan.n_multi < 2 * max(n_multi, 1)
            assert (plan.n_out == 0) == (n_out == 0) and n_out <= plan.n_out < max(2 * n_out, n_out + 16)
            seen.add((plan.n_tokens, plan.n_single, plan.n_multi))
    assert len({t for t, _, _ in seen}) == 8 + 6   # 16..128 in steps of 16, 192..512 in steps of 64


def test_wave_policy_admits_only_into_an_empty_engine():
    """The reference's comparator: nobody joins a running wave, a wave runs until its longest
    request has ended; a wave whose prompts the token budget cuts is admitted over several
    steps.  The tokens are those of continuous batching."""
    with pytest.raises(ValueError, match="policy"):
        make(n_pages=10, policy="waves")
    results = {}
    for policy in ("continuous", "wave"):
        sched, cache = make(n_pages=200, max_requests=3, max_batch_tokens=16, policy=policy)
        for i in range(7):
            sched.submit(Request(i, [i + 1] * (5 + i), greedy(2 + 3 * (i % 3))))
        log = []
        run(sched, cache, log)
        results[policy] = {i: sched.finished[i].generated for i in range(7)}
        first = {}
        last = {}
        for s, rows in enumerate(log):
            for rid, *_ in rows:
                first.setdefault(rid, s)
                last[rid] = s
        if policy == "wave":
            waves = [(0, 1, 2), (3, 4, 5), (6,)]
            for a, b in zip(waves, waves[1:]):
                assert max(last[i] for i in a) < min(first[i] for i in b)
            # prompts of 5, 6 and 7 tokens under a budget of 16: the third joins a step later
            assert first[0] == first[1] == 0 and first[2] in (0, 1)
            assert sched.stats.steps > results_steps
        else:
            results_steps = sched.stats.steps
            assert first[3] <= max(last[i] for i in (0, 1, 2))   # a freed slot is taken at once
    assert results["wave"] == results["continuous"]
    assert all(results["wave"][i] == oracle([i + 1] * (5 + i), greedy(2 + 3 * (i % 3)))
               for i in range(7))


def test_a_windowed_cache_needs_only_the_window(tmp_path):
    """A model whose cache groups all keep a window of keys: a request far longer than the pool
    is taken, because pages behind the window come back at every step; the same request is
    refused where every key is kept.  The reserve-full guard counts the window too."""
    page, window = 4, 10
    def build(win, n_pages, **kw):
        cache = CacheManager([KVSpec(1, 16, win)], [None], page, n_pages, 4)
        return Scheduler(cache, 1000, vocab_size=VOCAB, **kw), cache

    long_req = Request("long", list(range(60)), greedy(40))          # 99 cached tokens = 25 pages
    sched, cache = build(None, 8)
    with pytest.raises(ValueError, match="could never"):
        sched.submit(long_req)
    # window 10, one token per step: ceil(10 / 4) + 1 = 4 pages suffice
    assert cache.max_pages_held(99, 1) == [25]
    sched, cache = build(window, 4, max_batch_tokens=8)
    assert cache.max_pages_held(99, 1) == [4]
    sched.submit(long_req)
    run(sched, cache)
    assert sched.finished["long"].generated == oracle(long_req.prompt_ids, long_req.params)
    # reserve-full admission: two such requests fit a pool of 12 pages side by side (steps of up
    # to 8 tokens: ceil(17 / 4) + 1 = 6 pages each), which 2 x 25 pages never would
    sched, cache = build(window, 12, max_batch_tokens=8, admission="reserve_full")
    reqs = [Request(i, [(7 * i + j) % VOCAB for j in range(50)], greedy(30)) for i in range(2)]
    for r in reqs:
        sched.submit(r)
    log = []
    run(sched, cache, log)
    assert any(len({rid for rid, *_ in step}) == 2 for step in log)   # they ran side by side
    assert sched.stats.preemptions == 0
    for r in reqs:
        assert sched.finished[r.request_id].generated == oracle(r.prompt_ids, r.params)
