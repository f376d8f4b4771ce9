"""The cache manager: keys and values in pages with a block table per request, groups of
cache entries with different needs, and slots for per-request state of fixed size.

A *cache entry* is what one run of a layer caches (``ModelSpec.order`` numbers them).  Entries
whose mixers ask for the same :class:`KVSpec` (kv heads, head size, window) form a *group*: a
group has one page pool and one block table per request, and a page id is valid in every entry
of its group, as one block table serves all layers in the reference
(src/scratch_llm/kv_cache.py:326-333).  Groups whose mixers keep every key and groups that keep
a window of keys therefore have pages of their own; a window group gives pages back as soon as
the window has passed them.  Pages are given back when a request ends.  Page contents are
never cleared, not even once: nothing may depend on what a fresh or a reused page holds
(tests/test_paged_cache.py:164-184 of the reference poisons free blocks for the same reason;
``poison_free_pages=True`` does that here: the pool starts as NaN and every page that is given
back is filled with NaN again, so that a kernel that lets a stale place reach a result shows).

Beside the pages the manager owns ``max_requests`` *state slots*.  A request holds one slot
while it is live; entries whose mixer declares a :class:`StateSpec` get a tensor
``[max_requests, *shape]`` indexed by slot, zeroed when a request is admitted.  The Llama
architecture has no such state.  (A request's position and its sampling seed and counter live
on the host, with the scheduler, and are sent with every step's descriptor.)

The manager is host-side bookkeeping plus the device tensors; with ``device=None`` it allocates
no tensor and can be exercised on a machine without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..parts.base import KVSpec, StateSpec
from .pages import PagePool


@dataclass
class Group:
    spec: KVSpec
    entries: list[int]
    pool: PagePool
    pages: torch.Tensor | None = None  # [n_entries, n_pages, 2, kv_heads, page_size, head_dim]


@dataclass
class RequestCache:
    request_id: Hashable
    slot: int
    n_tokens: int = 0                      # tokens whose keys are cached (committed)
    n_reserved: int = 0                    # tokens that pages have been reserved for
    tables: list[list[int]] = field(default_factory=list)  # per group: logical -> physical, -1 freed
    # the same tables as int32 arrays (filled with -1 beyond the pages held), kept in step with
    # ``tables`` so that a step's descriptor copies rows instead of converting lists
    tables_np: list = field(default_factory=list)


class CacheManager:
    def __init__(self, kv_specs: Sequence[KVSpec | None],
                 state_specs: Sequence[StateSpec | None], page_size: int,
                 n_pages: int, max_requests: int, dtype: torch.dtype = torch.float32,
                 device: torch.device | str | None = None,
                 poison_free_pages: bool = False) -> None:
        if page_size < 1:
            raise ValueError(f"page size must be positive, got {page_size}")
        if max_requests < 1:
            raise ValueError("max_requests must be positive")
        self.page_size, self.max_requests = page_size, max_requests
        self.poison_free_pages = poison_free_pages
        self.dtype, self.device = dtype, (torch.device(device) if device is not None else None)
        self.groups: list[Group] = []
        self.entry_group: list[tuple[int, int] | None] = []  # entry -> (group, index in group)
        by_spec: dict[KVSpec, int] = {}
        for entry, spec in enumerate(kv_specs):
            if spec is None:
                self.entry_group.append(None)
                continue
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                self.groups.append(Group(spec, [], PagePool(n_pages)))
            g = by_spec[spec]
            self.entry_group.append((g, len(self.groups[g].entries)))
            self.groups[g].entries.append(entry)
        self.state_specs = list(state_specs)
        self.states: list[torch.Tensor | None] = [None] * len(self.state_specs)
        if self.device is not None:
            for group in self.groups:
                s = group.spec
                group.pages = torch.empty((len(group.entries), n_pages, 2, s.n_kv_heads,
                                           page_size, s.head_dim), dtype=dtype,
                                          device=self.device)
                if poison_free_pages:
                    group.pages.fill_(float("nan"))
            for entry, st in enumerate(self.state_specs):
                if st is not None:
                    self.states[entry] = torch.zeros((max_requests, *st.shape), dtype=st.dtype,
                                                     device=self.device)
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.requests: dict[Hashable, RequestCache] = {}

    # ------------------------------------------------------------------------- requests

    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, request_id: Hashable) -> RequestCache | None:
        """Give ``request_id`` a state slot; None if every slot is taken."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already live")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        rc = RequestCache(request_id, slot, tables=[[] for _ in self.groups],
                          tables_np=[np.full(16, -1, dtype=np.int32) for _ in self.groups])
        self.requests[request_id] = rc
        for state in self.states:
            if state is not None:
                state[slot].zero_()
        return rc

    def pages_needed(self, request_id: Hashable, n_new: int) -> list[int]:
        """Per group, how many pages must be added before ``n_new`` more tokens can be stored."""
        rc = self.requests[request_id]
        total = -(-(rc.n_tokens + n_new) // self.page_size)
        return [max(0, total - len(t)) for t in rc.tables]

    def max_pages_held(self, n_tokens: int, step_tokens: int = 1) -> list[int]:
        """Per group, the most pages a request holds at any time on its way to ``n_tokens``
        cached tokens when no step feeds it more than ``step_tokens``: all of them where every
        key is kept; where a window of w keys is kept, the pages that the window and one step's
        new tokens can touch (pages behind the window are given back at every commit)."""
        ps = self.page_size
        full = -(-n_tokens // ps)
        out = []
        for g in self.groups:
            w = g.spec.window
            out.append(full if w is None else
                       min(full, -(-(w - 1 + max(1, step_tokens)) // ps) + 1))
        return out

    def reserve(self, request_id: Hashable, n_new: int) -> bool:
        """Hold pages for the next ``n_new`` tokens in every group, or change nothing and
        return False if some group has too few free pages."""
        rc = self.requests[request_id]
        if rc.n_tokens + n_new <= rc.n_reserved and all(
                len(t) * self.page_size >= rc.n_tokens + n_new for t in rc.tables):
            return True   # an earlier call already holds the pages
        need = self.pages_needed(request_id, n_new)
        if any(n > g.pool.n_free for n, g in zip(need, self.groups)):
            return False
        for gi, (n, g, table) in enumerate(zip(need, self.groups, rc.tables)):
            got = g.pool.alloc(n, request_id)
            assert got is not None
            if n:
                arr = rc.tables_np[gi]
                if len(table) + n > arr.size:
                    grown = np.full(max(2 * arr.size, len(table) + n), -1, dtype=np.int32)
                    grown[:arr.size] = arr
                    arr = rc.tables_np[gi] = grown
                arr[len(table):len(table) + n] = got
            table.extend(got)
        rc.n_reserved = max(rc.n_reserved, rc.n_tokens + n_new)
        return True

    def commit(self, request_id: Hashable, n_new: int) -> None:
        """The step stored ``n_new`` tokens.  Window groups give back the pages that no later
        query can see: a query at position p sees keys j with p - window < j <= p, and the
        next query is at position n_tokens or later."""
        rc = self.requests[request_id]
        if rc.n_tokens + n_new > rc.n_reserved:
            raise ValueError(f"request {request_id!r}: {n_new} tokens stored but pages were "
                             f"reserved for {rc.n_reserved - rc.n_tokens}")
        rc.n_tokens += n_new
        for gi, (g, table) in enumerate(zip(self.groups, rc.tables)):
            if g.spec.window is None:
                continue
            last_dead = rc.n_tokens - g.spec.window  # positions <= last_dead are never read again
            n_dead_pages = max(0, (last_dead + 1) // self.page_size)
            dead = [table[i] for i in range(min(n_dead_pages, len(table))) if table[i] >= 0]
            if dead:
                self._give_back(g, dead, request_id)
                for i in range(min(n_dead_pages, len(table))):
                    table[i] = -1
                rc.tables_np[gi][:min(n_dead_pages, len(table))] = -1

    def release(self, request_id: Hashable) -> None:
        """The request has ended (or is set back): give its pages and its slot back."""
        rc = self.requests.pop(request_id)
        for g, table in zip(self.groups, rc.tables):
            self._give_back(g, [p for p in table if p >= 0], request_id)
        self._free_slots.append(rc.slot)

    def _give_back(self, group: Group, pages: list[int], request_id: Hashable) -> None:
        group.pool.free(pages, request_id)
        if self.poison_free_pages and pages and group.pages is not None:
            group.pages[:, torch.tensor(pages, device=group.pages.device)] = float("nan")

    # ---------------------------------------------------------------------------- views

    def table_of(self, request_id: Hashable, group: int) -> list[int]:
        return self.requests[request_id].tables[group]

    def table_array(self, request_id: Hashable, group: int) -> np.ndarray:
        """The block table as an int32 array of exactly the pages' count (a view)."""
        rc = self.requests[request_id]
        return rc.tables_np[group][:len(rc.tables[group])]

    def entry_pages(self, entry: int) -> tuple[torch.Tensor | None, int | None]:
        """(pages tensor of this entry, its group index)."""
        where = self.entry_group[entry]
        if where is None:
            return None, None
        g, i = where
        pages = self.groups[g].pages
        return (pages[i] if pages is not None else None), g

    def max_pages_per_request(self, max_position: int) -> int:
        return -(-max_position // self.page_size)

    # ---------------------------------------------------------------------------- stats

    def free_pages(self) -> list[int]:
        return [g.pool.n_free for g in self.groups]

    def waste_stats(self) -> dict[str, float]:
        """Allocated token places, live tokens and the unused fraction
        (src/scratch_llm/kv_cache.py:413-420 of the reference)."""
        allocated = live = 0
        for rc in self.requests.values():
            for g, table in zip(self.groups, rc.tables):
                held = sum(1 for p in table if p >= 0)
                allocated += held * self.page_size
                first_live = len(table) - held
                live += max(0, rc.n_tokens - first_live * self.page_size)
        return {"allocated_tokens": allocated, "live_tokens": live,
                "waste": 1.0 - live / allocated if allocated else 0.0}

    def check(self) -> None:
        """No page lost, held twice, or held by a request that is gone."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen: set[int] = set()
            for rc in self.requests.values():
                for p in rc.tables[gi]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise AssertionError(f"page {p} of group {gi} is in two block tables")
                    seen.add(p)
                    if g.pool.holder_of(p) != rc.request_id:
                        raise AssertionError(f"page {p} of group {gi} is in the table of "
                                             f"{rc.request_id!r} but held by "
                                             f"{g.pool.holder_of(p)!r}")
            if len(seen) != g.pool.n_held:
                raise AssertionError(f"group {gi}: {g.pool.n_held - len(seen)} held pages are "
                                     "in no block table")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice or is both free and held")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot was lost")
