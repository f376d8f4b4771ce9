"""Continuous batching: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees, and decides what happens when pages run out.

The reference's scheduler (src/scratch_llm/serving/continuous.py:91-409) runs admission
prefills and lockstep decodes as separate forwards, prefills one chunk of one request per
iteration in its chunked mode (:335-369), finishes on the budget only (:276-279), and cannot
run out of pages because it admits only what fits whole (:289-293).  Here every step is one
mixed batch:

1. every running request that is decoding gets its one token;
2. requests that are still reading their prompt get portions, oldest first, each
   ``min(rest of the prompt, chunk_size, budget left)``;
3. queued requests are admitted, first come first served, while a state slot, budget and
   pages for their first portion are there (``admission="reserve_full"`` instead admits only if
   the pool can hold every live request up to its full budget, the reference's guard).

**When pages run out** (only under ``admission="optimistic"``): a decoding request that cannot
get the page for its next token sets back the most recently admitted live request (possibly
itself): that request's pages and slot are freed, it returns to the front of the queue and is
later recomputed from its prompt plus the tokens it had generated, then goes on.  A prompt
portion that cannot get its pages is cut to what fits, or waits for a later step.  A request
that alone could never fit the pool is refused when it is submitted.

``policy="wave"`` is the reference's other policy (src/scratch_llm/serving/continuous.py:287,
449-476: requests are admitted only into an all-free batch, and a wave runs until its longest
request has finished), kept as the baseline that continuous batching is compared with: a wave
opens when no request is live, takes requests while slots, budget and pages allow (over several
steps if the token budget cuts its prompts), and closes when the slots are full or the queue is
empty.

The scheduler is host-side logic over a :class:`CacheManager`; it runs without a GPU.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Sequence

from ..cache import CacheManager
from ..sampling.params import SamplingParams


@dataclass
class Request:
    """One generation job (src/scratch_llm/serving/continuous.py:44-50 of the reference, plus
    sampling parameters; ``params.max_tokens`` is its max_new_tokens)."""

    request_id: Hashable
    prompt_ids: Sequence[int]
    params: SamplingParams = field(default_factory=lambda: SamplingParams(temperature=0.0))


@dataclass(eq=False)
class Sequence_:
    request: Request
    tokens: list[int]                 # prompt + generated so far
    n_prompt: int
    order: int = -1                   # admission counter; larger = admitted later
    logprobs: list[float] = field(default_factory=list)
    n_preempted: int = 0
    finish_reason: str | None = None
    admitted_at_step: int = -1

    @property
    def generated(self) -> list[int]:
        return self.tokens[self.n_prompt:]


@dataclass(eq=False)
class PlannedRow:
    seq: Sequence_
    start: int        # index of the first token fed (= tokens cached before the step)
    n: int            # how many tokens are fed
    samples: bool     # True if the row's last token is the sequence's last: logits wanted


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    stalled_portions: int = 0
    peak_live: int = 0
    rows_per_step: list[int] = field(default_factory=list)
    tokens_per_step: list[int] = field(default_factory=list)
    page_occupancy: list[float] = field(default_factory=list)
    # what the held pages waste (the reference's paged_frag_mean and paged_alloc_peak_tokens,
    # src/scratch_llm/serving/continuous.py:67-87), sampled every WASTE_EVERY steps before
    # finished requests give their pages back
    waste_samples: list[float] = field(default_factory=list)
    allocated_peak_tokens: int = 0

    @property
    def waste_mean(self) -> float | None:
        return sum(self.waste_samples) / len(self.waste_samples) if self.waste_samples else None


#: the cache's waste is sampled every so many steps (it walks every live request's tables)
WASTE_EVERY = 8


class Scheduler:
    def __init__(self, cache: CacheManager, max_position: int, max_batch_tokens: int = 2048,
                 chunk_size: int | None = None, admission: str = "optimistic",
                 vocab_size: int | None = None, policy: str = "continuous") -> None:
        if admission not in ("optimistic", "reserve_full"):
            raise ValueError("admission is 'optimistic' or 'reserve_full'")
        if policy not in ("continuous", "wave"):
            raise ValueError("policy is 'continuous' or 'wave'")
        self.policy = policy
        self._wave_open = True
        if max_batch_tokens < 1 or (chunk_size is not None and chunk_size < 1):
            raise ValueError("max_batch_tokens and chunk_size must be positive")
        self.cache, self.max_position = cache, max_position
        self.max_batch_tokens, self.chunk_size = max_batch_tokens, chunk_size
        self.admission, self.vocab_size = admission, vocab_size
        self.queue: deque[Sequence_] = deque()
        self.running: list[Sequence_] = []      # in admission order
        self.finished: dict[Hashable, Sequence_] = {}
        self.stats = SchedulerStats()
        self._admissions = 0
        self._known: set[Hashable] = set()

    # ---------------------------------------------------------------------------- submit

    def _pool_pages(self) -> list[int]:
        return [g.pool.n_pages for g in self.cache.groups]

    def _pages_by_last_token(self, n_prompt: int, max_tokens: int, step_tokens: int) -> list[int]:
        """Per cache group, the most pages a request holds on its way to its last token (the
        cache manager knows which groups keep every key and which a window of them)."""
        return self.cache.max_pages_held(n_prompt + max_tokens - 1, step_tokens)

    def submit(self, request: Request) -> None:
        prompt = list(request.prompt_ids)
        p = request.params
        if request.request_id in self._known:
            raise ValueError(f"request id {request.request_id!r} was already submitted")
        if not prompt:
            raise ValueError("prompt_ids must be non-empty")
        if self.vocab_size is not None and not all(0 <= t < self.vocab_size for t in prompt):
            raise ValueError(f"prompt token out of range [0, {self.vocab_size})")
        if len(prompt) + p.max_tokens > self.max_position:
            raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({p.max_tokens}) exceeds "
                             f"max_position {self.max_position}")
        # (fed one token per step if need be: portions are cut to the pages that are free)
        need = self._pages_by_last_token(len(prompt), p.max_tokens, 1)
        if any(n > have for n, have in zip(need, self._pool_pages())):
            raise ValueError(f"request {request.request_id!r} needs {need} pages by its last "
                             f"token but the pool has {self._pool_pages()} (per cache group): "
                             "it could never finish")
        self._known.add(request.request_id)
        self.queue.append(Sequence_(request, prompt, len(prompt)))

    @property
    def has_work(self) -> bool:
        return bool(self.queue or self.running)

    # ------------------------------------------------------------------------------ plan

    def _cached(self, seq: Sequence_) -> int:
        return self.cache.requests[seq.request.request_id].n_tokens

    def _preempt(self, seq: Sequence_) -> None:
        self.cache.release(seq.request.request_id)
        self.running.remove(seq)
        seq.n_preempted += 1
        self.queue.appendleft(seq)
        self.stats.preemptions += 1

    def _fits(self, seq: Sequence_, n: int) -> int:
        """The largest m <= n for which pages can be reserved now (0 if none)."""
        rid = seq.request.request_id
        if self.cache.reserve(rid, n):
            return n
        rc = self.cache.requests[rid]
        ps = self.cache.page_size
        room = min((len(t) + g.pool.n_free) * ps for t, g in zip(rc.tables, self.cache.groups))
        m = min(n, room - rc.n_tokens)
        if m >= 1 and self.cache.reserve(rid, m):
            return m
        return 0

    def _step_cap(self) -> int:
        return min(self.max_batch_tokens, self.chunk_size or self.max_batch_tokens)

    def _committed_pages(self) -> list[int]:
        """Per group, what the live requests may come to hold by their last tokens."""
        total = [0] * len(self.cache.groups)
        for s in self.running:
            need = self._pages_by_last_token(s.n_prompt, s.request.params.max_tokens,
                                             self._step_cap())
            total = [a + b for a, b in zip(total, need)]
        return total

    def plan(self) -> list[PlannedRow]:
        """Decide the next step's batch.  Reserves the pages its rows need."""
        budget = self.max_batch_tokens
        rows: list[PlannedRow] = []
        planned: set[int] = set()      # id() of the sequences that have a row in this step
        gone: set[int] = set()         # id() of the sequences set back while planning
        # 1. decoding requests, oldest first; a page shortage sets back the newest request
        for seq in list(self.running):
            if id(seq) in gone:        # set back while serving an older one
                continue
            cached = self._cached(seq)
            if cached != len(seq.tokens) - 1 or budget < 1:
                continue
            rid = seq.request.request_id
            while not self.cache.reserve(rid, 1):
                victim = max(self.running, key=lambda s: s.order)
                if id(victim) in planned:
                    for r in [r for r in rows if r.seq is victim]:
                        rows.remove(r)
                        budget += r.n
                    planned.discard(id(victim))
                self._preempt(victim)
                gone.add(id(victim))
                if victim is seq:
                    break
            else:
                rows.append(PlannedRow(seq, cached, 1, True))
                planned.add(id(seq))
                budget -= 1
        # 2. prompts in progress, oldest first
        for seq in self.running:
            if id(seq) in planned or budget < 1:
                continue
            cached = self._cached(seq)
            rest = len(seq.tokens) - cached
            if rest < 1:
                continue
            n = min(rest, budget, self.chunk_size or rest)
            m = self._fits(seq, n)
            if m == 0:
                self.stats.stalled_portions += 1
                continue
            rows.append(PlannedRow(seq, cached, m, cached + m == len(seq.tokens)))
            planned.add(id(seq))
            budget -= m
        # 3. admissions, first come first served, no skipping ahead
        if self.policy == "wave":
            if not self.running:
                self._wave_open = True
            elif not self._wave_open:
                budget = 0          # a wave is running: nobody joins it
        while self.queue and budget >= 1 and self.cache.n_free_slots > 0:
            seq = self.queue[0]
            if self.admission == "reserve_full":
                need = self._pages_by_last_token(seq.n_prompt, seq.request.params.max_tokens,
                                                 self._step_cap())
                if any(c + n > have for c, n, have in
                       zip(self._committed_pages(), need, self._pool_pages())):
                    break
            n = min(len(seq.tokens), budget, self.chunk_size or len(seq.tokens))
            rid = seq.request.request_id
            assert self.cache.admit(rid) is not None
            m = self._fits(seq, n)
            if m == 0:
                self.cache.release(rid)
                break
            self.queue.popleft()
            seq.order = self._admissions
            self._admissions += 1
            if seq.admitted_at_step < 0:
                seq.admitted_at_step = self.stats.steps
            self.running.append(seq)
            rows.append(PlannedRow(seq, 0, m, m == len(seq.tokens)))
            budget -= m
        if self.policy == "wave" and self._wave_open and self.running and \
                (not self.queue or self.cache.n_free_slots == 0):
            self._wave_open = False     # full, or nobody left to take: the wave is closed
        # nothing can move although requests are live: the pool is full of half-read prompts
        if not rows and self.running:
            victim = max(self.running, key=lambda s: s.order)
            if len(self.running) == 1:
                raise RuntimeError("a single live request cannot get pages: the pool is too "
                                   "small for it")
            self._preempt(victim)
            return self.plan()
        return rows

    def plan_ahead(self, in_flight: Sequence[PlannedRow]) -> list[tuple[PlannedRow, int]] | None:
        """The step after ``in_flight``, planned while ``in_flight`` still runs and its tokens
        are unknown: every live request decodes the token it is about to get.  Returns rows with,
        for each, the place of its request among the sampling rows of ``in_flight`` (where its
        pending token will lie), or None if the next step is not that simple (requests are
        queued, a prompt is half read, pages are short): then :meth:`plan` decides, after
        :meth:`complete`.  A request that its pending token ends for certain (length) is left
        out; one that it may end (a stop token) is planned, and its row is dropped by
        :meth:`complete` if it did end."""
        if self.queue or not self.running:
            return None
        place: dict[int, int] = {}
        k = 0
        for r in in_flight:
            if r.samples:
                place[id(r.seq)] = k
                k += 1
        chosen: list[tuple[Sequence_, int]] = []
        for seq in self.running:
            j = place.get(id(seq))
            if j is None:
                return None
            after = len(seq.tokens) + 1        # with the pending token
            if after - seq.n_prompt >= seq.request.params.max_tokens or after >= self.max_position:
                continue
            chosen.append((seq, j))
        if not chosen or len(chosen) > self.max_batch_tokens:
            return None
        for seq, _ in chosen:
            if not self.cache.reserve(seq.request.request_id, 1):
                return None
        return [(PlannedRow(seq, self._cached(seq), 1, True), j) for seq, j in chosen]

    # -------------------------------------------------------------------------- complete

    def commit_rows(self, rows: Sequence[PlannedRow]) -> None:
        """What the step function does after it stored the rows' keys and values; for callers
        that stand in for the step function."""
        for r in rows:
            self.cache.commit(r.seq.request.request_id, r.n)

    def complete(self, rows: Sequence[PlannedRow], sampled: Sequence[int],
                 logprobs: Sequence[float] | None = None) -> list[Sequence_]:
        """The step ran (and committed its tokens to the cache): ``sampled`` holds one token
        for every row with ``samples`` set, in order.  Returns the sequences that finished."""
        done: list[Sequence_] = []
        k = 0
        st = self.stats
        st.steps += 1
        st.rows_per_step.append(len(rows))
        st.tokens_per_step.append(sum(r.n for r in rows))
        st.peak_live = max(st.peak_live, len(self.running))
        if st.steps % WASTE_EVERY == 1:
            waste = self.cache.waste_stats()
            st.waste_samples.append(waste["waste"])
            st.allocated_peak_tokens = max(st.allocated_peak_tokens, int(waste["allocated_tokens"]))
        for r in rows:
            rid = r.seq.request.request_id
            if r.seq.finish_reason:
                pass
            elif r.n == 1 and r.start >= r.seq.n_prompt:
                st.decode_tokens += 1
            else:
                st.prefill_tokens += r.n
            if not r.samples:
                continue
            token = int(sampled[k])
            k += 1
            seq = r.seq
            if seq.finish_reason:        # planned ahead, and the token before this one ended it
                continue
            if logprobs is not None:
                seq.logprobs.append(float(logprobs[k - 1]))
            seq.tokens.append(token)
            p = seq.request.params
            if token in p.stop_ids:
                seq.finish_reason = "stop"       # the stop token is kept in the output
            elif len(seq.generated) >= p.max_tokens:
                seq.finish_reason = "length"
            elif len(seq.tokens) >= self.max_position:
                seq.finish_reason = "max_position"
            if seq.finish_reason:
                self.cache.release(rid)
                self.running.remove(seq)
                self.finished[rid] = seq
                done.append(seq)
        if self.cache.groups:
            g = self.cache.groups[0]
            st.page_occupancy.append(1.0 - g.pool.n_free / g.pool.n_pages)
        return done
