"""The Python entry point: a model folder in, generated token ids out.

The reference's entry points are ``generate(model, prompt_ids, params, device, use_cache)``
returning the generated ids only (src/scratch_llm/sampling.py:185-204),
``generate_with_logprobs`` (:207-217) and ``serve_continuous(model, requests, n_slots, ...)``
returning completed requests with their tokens (src/scratch_llm/serving/continuous.py:412-446).
:class:`LLM` offers the same three on top of the scheduler and the step function; host token
ids go in, host token ids come out.
"""

from __future__ import annotations

import time
import zlib
from dataclasses import dataclass
from pathlib import Path
from typing import Hashable, Sequence

import torch

from ..kernels import ops
from ..sampling import Sampler, SamplingParams
from ..sampling.sampler import PendingSample
from .batch import RowInput
from .runner import ModelRunner, load_model
from .scheduler import PlannedRow, Request, Scheduler, SchedulerStats, Sequence_


@dataclass(frozen=True)
class Completed:
    """A finished request (src/scratch_llm/serving/continuous.py:53-66 of the reference)."""

    request: Request
    token_ids: tuple[int, ...]
    logprobs: tuple[float, ...] | None
    finish_reason: str
    admitted_at_step: int
    n_preempted: int
    #: when the request arrived and when the host had each of its tokens, on ``serve``'s clock
    #: (the reference's RequestRecord: start_s, token_times_s)
    start_s: float = 0.0
    token_times_s: tuple[float, ...] = ()


@dataclass(frozen=True)
class ServeResult:
    completed: tuple[Completed, ...]   # in the order the requests were given
    stats: SchedulerStats
    wall_s: float


@dataclass
class _InFlight:
    """A step that was launched and whose tokens the host has not read yet."""

    rows: list[PlannedRow]
    sampling: list[Sequence_]
    pending: PendingSample | None


#: :meth:`LLM.step` reads the kernels' error words every this many steps
CHECK_ERRORS_EVERY = 128


def _seed_of(request: Request) -> int:
    if request.params.seed is not None:
        return int(request.params.seed)
    return zlib.crc32(repr(request.request_id).encode("utf-8"))


class LLM:
    """``max_tokens`` is the cache capacity in tokens (the page pool holds that many);
    ``page_size`` the tokens of a cache page (64 by default: the tcgen05 attention fetches keys
    and values with one TMA request per page and 64-column block, and with 16-token pages the
    number of requests, not the arithmetic, set its speed: 73.5 against 61.5 us at 2,048 tokens);
    ``max_requests`` the number of requests that can be live at once; ``max_batch_tokens`` the
    token budget of one step; ``chunk_size`` the largest prompt portion per request and step
    (None: the budget alone cuts prompts).

    ``lookahead``: while a decode step runs, the next one is planned, packed and launched with
    its input tokens still on the device (the sampler's output feeds the embedding directly), and
    only then does the host wait for the tokens of the first.  The device then never waits for
    the host between decode steps.  What a step computes does not change; a request that a stop
    token ends has one more row in flight, whose result is dropped."""

    def __init__(self, model: str | Path, dtype: str = "bfloat16", max_tokens: int = 65536,
                 page_size: int = 64, max_requests: int = 64, max_batch_tokens: int = 2048,
                 chunk_size: int | None = None, admission: str = "optimistic",
                 verbose: bool = False, lookahead: bool = True) -> None:
        self.model = load_model(model, dtype, verbose=verbose) if isinstance(model, (str, Path)) \
            else model
        self.runner = ModelRunner(self.model, page_size, max(1, -(-max_tokens // page_size)),
                                  max_requests)
        self.sampler = Sampler(self.runner.device)
        self.max_batch_tokens, self.chunk_size, self.admission = (max_batch_tokens, chunk_size,
                                                                  admission)
        self._sched: Scheduler | None = None
        self.lookahead = lookahead
        self._in_flight: _InFlight | None = None
        self._unchecked_steps = 0

    def _scheduler(self, policy: str = "continuous") -> Scheduler:
        return Scheduler(self.runner.cache, self.runner.max_position, self.max_batch_tokens,
                         self.chunk_size, self.admission, self.runner.vocab_size, policy)

    # ------------------------------------------------------------------- submit and step

    def submit(self, request: Request) -> None:
        """Queue a request; :meth:`step` runs it."""
        if self._sched is None:
            self._sched = self._scheduler()
        self._sched.submit(request)

    @property
    def has_work(self) -> bool:
        return self._sched is not None and self._sched.has_work

    def _launch(self, rows: list[PlannedRow], places: Sequence[int] | None,
                want_logprobs: bool) -> "_InFlight":
        """Run ``rows`` and choose their next tokens, without waiting for either.  ``places``:
        for rows planned ahead, where each row's input token lies in the pending buffer."""
        if places is None:
            inputs = [RowInput(r.seq.request.request_id, r.seq.tokens[r.start:r.start + r.n],
                               [r.n - 1] if r.samples else []) for r in rows]
        else:
            inputs = [RowInput(r.seq.request.request_id, [0], [0], pending=j)
                      for r, j in zip(rows, places)]
        ahead = 0 if places is None else 1     # tokens of the request the host has not seen
        logits = self.runner.step(inputs)
        sampling = [r.seq for r in rows if r.samples]
        pending = None
        if sampling:
            pending = self.sampler.sample_async(
                logits, [s.request.params for s in sampling],
                [_seed_of(s.request) for s in sampling],
                [len(s.generated) + ahead for s in sampling], want_logprobs,
                out=self.runner.pending_tokens[:len(sampling)])
        return _InFlight(rows, sampling, pending)

    @torch.no_grad()
    def step(self, want_logprobs: bool = False) -> dict[Hashable, int]:
        """One scheduler step: plan a batch, run it, choose the next tokens.  Returns the token
        each request produced in this step ({request id: token}, on the host)."""
        sched = self._sched
        cur = self._in_flight
        if cur is None:
            cur = self._launch(sched.plan(), None, want_logprobs)
        self._in_flight = None
        if self.lookahead and cur.pending is not None:
            ahead = sched.plan_ahead(cur.rows)
            if ahead is not None:
                self._in_flight = self._launch([r for r, _ in ahead], [j for _, j in ahead],
                                               want_logprobs)
        tokens, lps = cur.pending.result() if cur.pending is not None else ([], None)
        # kernels with bounded waits record a code and go on with invalid results when a wait
        # gives up: reading the codes waits for the device, so they are read every so many
        # steps (and at the end of serve), and the error is raised before more tokens are kept
        self._unchecked_steps += 1
        if self._unchecked_steps >= CHECK_ERRORS_EVERY:
            self._unchecked_steps = 0
            ops.check_kernel_errors()
        alive = [not s.finish_reason for s in cur.sampling]
        sched.complete(cur.rows, tokens, lps)
        return {s.request.request_id: t for s, t, a in zip(cur.sampling, tokens, alive) if a}

    def abort_all(self) -> None:
        """Drop every queued and live request and give back what they hold."""
        self._in_flight = None
        if self._sched is not None:
            for seq in list(self._sched.running):
                self.runner.cache.release(seq.request.request_id)
        self._sched = None

    # ------------------------------------------------------------------------------ serve

    def serve(self, requests: Sequence[Request], want_logprobs: bool = False, *,
              arrivals_s: Sequence[float] | None = None, clock=time.perf_counter,
              sleep=time.sleep, policy: str = "continuous") -> ServeResult:
        """Run ``requests`` to completion under continuous batching.  ``arrivals_s`` (one
        offset in seconds per request, from the start of the call) turns the closed list into a
        stream: a request is queued once ``clock`` has passed its offset, and ``sleep`` is the
        idle wait while nothing is live (both can be replaced, for a test's own clock), as in the
        reference's ``serve`` (src/scratch_llm/serving/continuous.py:98-121, 268-274).
        ``policy="wave"``: requests join only when no request is live (the reference's baseline)."""
        if self.has_work:
            raise RuntimeError("serve() needs an idle engine: requests from submit() are live")
        n = len(requests)
        if arrivals_s is not None:
            if len(arrivals_s) != n:
                raise ValueError("arrivals_s must carry one offset per request")
            if any(a < 0 for a in arrivals_s):
                raise ValueError("arrivals_s offsets must be >= 0 (they are offsets from the start)")
        arrival = [float(a) for a in arrivals_s] if arrivals_s is not None else [0.0] * n
        waiting = sorted(range(n), key=lambda i: (arrival[i], i))
        waiting.reverse()   # the next arrival last, to pop it
        times: dict[Hashable, list[float]] = {r.request_id: [] for r in requests}
        self._sched = self._scheduler(policy)
        start = time.perf_counter()
        t0 = clock()
        try:
            while waiting or self.has_work:
                while waiting and clock() - t0 >= arrival[waiting[-1]]:
                    self.submit(requests[waiting.pop()])
                if not self.has_work:
                    sleep(max(0.0, t0 + arrival[waiting[-1]] - clock()))
                    continue
                produced = self.step(want_logprobs)
                now = clock()
                for rid in produced:
                    times[rid].append(now)
            sched = self._sched
            self._in_flight = None   # rows planned ahead for requests that have all ended
            ops.check_kernel_errors()
        except BaseException:
            self.abort_all()   # an error leaves nothing held
            raise
        self._sched = None
        wall = time.perf_counter() - start
        done = []
        for i, r in enumerate(requests):
            seq: Sequence_ = sched.finished[r.request_id]
            done.append(Completed(r, tuple(seq.generated),
                                  tuple(seq.logprobs) if want_logprobs else None,
                                  seq.finish_reason or "", seq.admitted_at_step, seq.n_preempted,
                                  t0 + arrival[i], tuple(times[r.request_id])))
        return ServeResult(tuple(done), sched.stats, wall)

    # --------------------------------------------------------------------------- generate

    def generate(self, prompts, params: SamplingParams | Sequence[SamplingParams] | None = None):
        """Generated token ids (without the prompt; a stop token is included) for one prompt
        (a list of ints -> a list of ints) or several (a list of lists -> a list of lists)."""
        return self._generate(prompts, params, False)[0]

    def generate_with_logprobs(self, prompts, params=None):
        """Like :meth:`generate`, and each token's log-probability under the raw model
        distribution at temperature 1."""
        return self._generate(prompts, params, True)

    def _generate(self, prompts, params, want_logprobs):
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        if params is None:
            params = SamplingParams()
        pl = [params] * len(plist) if isinstance(params, SamplingParams) else list(params)
        if len(pl) != len(plist):
            raise ValueError("one SamplingParams per prompt, or one for all")
        result = self.serve([Request(i, p, sp) for i, (p, sp) in enumerate(zip(plist, pl))],
                            want_logprobs)
        toks = [list(c.token_ids) for c in result.completed]
        lps = [list(c.logprobs) for c in result.completed] if want_logprobs else None
        if single:
            return toks[0], (lps[0] if lps else None)
        return toks, lps

    # ------------------------------------------------------------------------------ score

    @torch.no_grad()
    def _response_rows(self, prompt_ids: Sequence[int], response_ids: Sequence[int],
                       whole_rows: bool):
        """The rows that predict each response token (position p-1+i predicts response token i),
        through the step function in portions of at most the token budget: the taken tokens'
        log-probabilities [T], or the whole log_softmax rows [T, vocab] on the device."""
        prompt, resp = list(prompt_ids), list(response_ids)
        if not prompt or not resp:
            raise ValueError("score needs a non-empty prompt and a non-empty response")
        if self.has_work:
            raise RuntimeError("score() needs an idle engine: requests from submit() are live")
        tokens = (prompt + resp)[:-1]       # the last response token predicts nothing asked for
        first = len(prompt) - 1
        rid = ("score", id(tokens))
        runner = self.runner
        if not runner.admit(rid):
            raise RuntimeError("no free request slot")
        out = []
        try:
            for a in range(0, len(tokens), self.max_batch_tokens):
                part = tokens[a:a + self.max_batch_tokens]
                want = [i for i in range(len(part)) if a + i >= first]
                logits = runner.step([RowInput(rid, part, want)])
                if not want:
                    continue
                if whole_rows:
                    rows = torch.empty_like(logits)
                    ops.log_softmax(logits, rows_out=rows)
                    out.append(rows)
                else:
                    taken = torch.tensor([resp[a + i - first] for i in want], dtype=torch.int32,
                                         device=logits.device)
                    lp = torch.empty(len(want), dtype=torch.float32, device=logits.device)
                    ops.log_softmax(logits, taken=taken, taken_out=lp)
                    out.append(lp)
        finally:
            runner.release(rid)
        return torch.cat(out)

    def score(self, prompt_ids, response_ids):
        """Log-probabilities of the given response tokens under the model at temperature 1, one
        forward over prompt + response (the reference's ``LocalBackend.score``,
        src/scratch_llm/rollout/local.py:50-62).  One pair (lists of ints -> a list of floats)
        or several (lists of lists -> a list of lists)."""
        if len(prompt_ids) > 0 and isinstance(prompt_ids[0], int):
            return self._response_rows(prompt_ids, response_ids, False).tolist()
        if len(prompt_ids) != len(response_ids):
            raise ValueError("one response per prompt")
        return [self._response_rows(p, r, False).tolist()
                for p, r in zip(prompt_ids, response_ids)]

    def distribution_logprobs(self, prompt_ids: Sequence[int], response_ids: Sequence[int]
                              ) -> torch.Tensor:
        """The whole log_softmax rows [len(response), vocab] at the response positions, on the
        device (the reference's ``LocalBackend.distribution_logprobs``,
        src/scratch_llm/rollout/local.py:64-70)."""
        return self._response_rows(prompt_ids, response_ids, True)


def generate(llm: LLM, prompt_ids: Sequence[int], params: SamplingParams) -> list[int]:
    """The reference's ``generate`` with the engine in the model's place."""
    return llm.generate(list(prompt_ids), params)


def generate_with_logprobs(llm: LLM, prompt_ids: Sequence[int], params: SamplingParams
                           ) -> tuple[list[int], list[float]]:
    return llm.generate_with_logprobs(list(prompt_ids), params)


def serve_continuous(llm: LLM, requests: Sequence[Request], *,
                     arrivals_s: Sequence[float] | None = None, clock=time.perf_counter,
                     sleep=time.sleep) -> ServeResult:
    return llm.serve(requests, arrivals_s=arrivals_s, clock=clock, sleep=sleep)


def serve_static_wave(llm: LLM, requests: Sequence[Request], *, clock=time.perf_counter
                      ) -> ServeResult:
    """The reference's comparator (src/scratch_llm/serving/continuous.py:449-476): requests are
    admitted only when no request is live, a wave runs until its longest request has ended."""
    return llm.serve(requests, clock=clock, policy="wave")


def batched_greedy_decode(llm: LLM, prompts: Sequence[Sequence[int]], max_tokens: int
                          ) -> list[list[int]]:
    """The reference's static batched decode (src/scratch_llm/serving/batched.py:26-58) with the
    engine in the model's place: the generated ids of every prompt, greedy, exactly
    ``max_tokens`` each (no stop ids).  The reference needs prompts of one length, because its
    rows share their positions; here every row has its own, so any lengths are taken."""
    if len(prompts) == 0:
        raise ValueError("prompts must be non-empty")
    return llm.generate([list(p) for p in prompts],
                        SamplingParams(temperature=0.0, max_tokens=max_tokens))
