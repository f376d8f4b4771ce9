"""The batch of one step: a packed list of rows, each row the next tokens of one request.

Rows may be portions of prompts (of any length, cut anywhere) beside single decoded tokens, in
any order.  The reference has three separate forward modes chosen by the cache object's type
(src/scratch_llm/model.py:290-325, 493-498) and never mixes them; here one descriptor covers
all of them:

=============  ======================  ==================================================
token_ids      int32 [n_tokens]        all rows' new tokens, row after row
positions      int32 [n_tokens]        absolute position of each token in its request
token_row      int32 [n_tokens]        row of each token
row_start      int32 [n_rows + 1]      offset of each row's first token (cu_seqlens)
row_pos0       int32 [n_rows]          position of each row's first new token
row_slot       int32 [n_rows]          the request's state slot
block_tables   int32 [n_rows, P] each  per cache group: physical page of each logical page
logit_index    int32 [n_out]           flat token indices whose logits are wanted
=============  ======================  ==================================================

All of it is packed on the host into one pinned buffer and reaches the device in one copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class PadPlan:
    """The sizes a small step is padded to, so that steps of many shapes share few captured
    graphs.  Padding tokens follow the last row's tokens: id 0, position 0, ``token_row`` -1
    (they belong to no row, nothing of them is stored and attention skips them).  Padding rows
    have no tokens; the lists of single and multi rows are filled up with such a row."""

    n_tokens: int
    n_single: int
    n_multi: int
    n_out: int


#: steps of up to this many tokens are padded and replayed as graphs; larger ones keep the
#: device busy for longer than the host needs to launch them
PAD_MAX_TOKENS = 512


def _round_up(n: int, step: int) -> int:
    return -(-n // step) * step


def _next_power_of_two(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def pad_plan(n_tokens: int, n_single: int, n_multi: int, n_out: int) -> PadPlan:
    """Tokens go up to a multiple of 16 (of 64 above 128), single rows to a multiple of 8,
    multi rows to a power of two, wanted places to a power of two up to 8 and to a multiple of
    16 above; nothing wanted stays nothing wanted.  A decode step (every row one token, its
    logits wanted) only goes up to the next multiple of 8 (of 16 above 32 rows, of 32 above 64)
    in all three."""
    if n_multi == 0 and n_tokens == n_single == n_out:
        # (rows of padding cost a decode step next to nothing, a shape that has not come before
        # costs a capture: the steps get coarser as the batch grows)
        n = _round_up(n_tokens, 8 if n_tokens <= 32 else 16 if n_tokens <= 64 else 32)
        return PadPlan(n, n, 0, n)
    tokens = _round_up(n_tokens, 16) if n_tokens <= 128 else _round_up(n_tokens, 64)
    out = 0 if n_out == 0 else _next_power_of_two(n_out) if n_out <= 8 else _round_up(n_out, 16)
    return PadPlan(tokens, _round_up(n_single, 8), _next_power_of_two(n_multi) if n_multi else 0,
                   out)


@dataclass
class RowInput:
    """The next tokens of one request and the places among them whose logits are wanted."""

    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    #: the row's one token is not on the host yet: it is entry ``pending`` of the device buffer
    #: that the step is given (``tokens`` then holds one placeholder)
    pending: int | None = None


@dataclass
class StepBatch:
    n_tokens: int
    n_rows: int
    n_out: int
    max_new: int
    max_context: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_row: torch.Tensor
    row_start: torch.Tensor
    row_pos0: torch.Tensor
    row_slot: torch.Tensor
    logit_index: torch.Tensor
    block_tables: list[torch.Tensor] = field(default_factory=list)
    # rows with exactly one new token (decode) and rows with several (prompt portions), as
    # device lists, with what a part needs to plan its launches for them
    single_rows: torch.Tensor | None = None
    multi_rows: torch.Tensor | None = None
    # tokens chosen on the device that the host has not read yet (ids -1 - j in token_ids)
    pending_tokens: torch.Tensor | None = None
    n_single: int = 0
    n_multi: int = 0
    max_new_multi: int = 0
    max_context_single: int = 0
    context_bucket: int = 0   # max_context_single rounded up to a power of two (at least 256)
    #: the logits of every token are wanted, in the tokens' order (a decode step: the gather of
    #: the wanted rows before the final norm is then the identity)
    wants_every_token: bool = False
    # host copies, for parts that plan their launches from them
    host_row_new: list[int] = field(default_factory=list)
    host_row_pos0: list[int] = field(default_factory=list)
    # a padded step (see PadPlan): tokens and wanted places that are real; the sizes above
    # count the padding, and max_new / max_new_multi are then upper bounds
    padded: bool = False
    n_real_tokens: int = 0
    n_real_out: int = 0


class BatchStager:
    """Packs step descriptors on the host and copies them to the device in one transfer.
    Two pinned buffers alternate, each guarded by an event, so that packing step n+1 never
    overwrites bytes that step n's copy is still reading."""

    def __init__(self, device: torch.device, capacity_ints: int = 1 << 16) -> None:
        self.device = device
        self._turn = 0
        self.bytes_uploaded = 0   # host-to-device bytes so far
        self._allocate(capacity_ints)

    def _allocate(self, n: int) -> None:
        self._host = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._host_np = [h.numpy() for h in self._host]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._dev = torch.empty(n, dtype=torch.int32, device=self.device)
        # per tuple of array shapes: offsets, total, the device views and the slices to copy.
        # Decode steps repeat their shapes, and making a dozen tensor views costs more host
        # time than packing the arrays.
        self._layouts: dict[tuple, tuple] = {}

    def reserve(self, n: int) -> None:
        """Make room for ``n`` ints now, so that later uploads keep their device addresses."""
        if n > self._dev.numel():
            self._grow(n)

    def _grow(self, n: int) -> None:
        cap = self._dev.numel()
        while cap < n:
            cap *= 2
        torch.cuda.current_stream().synchronize()
        self._allocate(cap)

    def _layout(self, shapes: tuple) -> tuple:
        offsets, total = [], 0
        for shape in shapes:
            size = int(np.prod(shape))
            offsets.append((total, size))
            total += (size + 3) // 4 * 4
        if total > self._dev.numel():
            self._grow(total)
        views = [self._dev[o:o + size].view(shape) for (o, size), shape in zip(offsets, shapes)]
        layout = (offsets, total, views, self._dev[:total], [h[:total] for h in self._host])
        self._layouts[shapes] = layout
        return layout

    def upload(self, parts: Sequence[np.ndarray]) -> list[torch.Tensor]:
        """Copy the int32 arrays to the device; returns one device view per array (each view
        starts on a 16-byte boundary).  The views of equal shapes are the same tensors from
        call to call: they are valid until the next upload."""
        shapes = tuple(a.shape for a in parts)
        layout = self._layouts.get(shapes) or self._layout(shapes)
        offsets, total, views, dev_slice, host_slices = layout
        turn = self._turn
        self._turn ^= 1
        self._events[turn].synchronize()   # the copy that last read this buffer is done
        hnp = self._host_np[turn]
        for a, (o, size) in zip(parts, offsets):
            hnp[o:o + size] = a.reshape(-1)
        if total:
            dev_slice.copy_(host_slices[turn], non_blocking=True)
            self.bytes_uploaded += 4 * total
        self._events[turn].record()
        return list(views)


def context_bucket(context: int) -> int:
    bucket = 256
    while bucket < context:
        bucket *= 2
    return bucket


def build_batch(cache, stager: BatchStager, rows: Sequence[RowInput], vocab_size: int,
                max_position: int, table_width: int | None = None,
                pad: bool = False) -> StepBatch:
    """Check the rows against the cache manager's view of their requests, pack the descriptor
    and copy it to the device.  ``table_width`` fixes the width of the block tables (for a
    step that replays a captured CUDA graph, every array must keep its size and address).
    ``pad``: bring the step to the sizes of :func:`pad_plan`."""
    n_rows = len(rows)
    lens = [len(r.tokens) for r in rows]
    if n_rows and min(lens) < 1:
        bad = rows[lens.index(min(lens))]
        raise ValueError(f"request {bad.request_id!r}: a row needs at least one token")
    if len({r.request_id for r in rows}) != n_rows:
        seen: set[Hashable] = set()
        for r in rows:
            if r.request_id in seen:
                raise ValueError(f"request {r.request_id!r} appears twice in one step")
            seen.add(r.request_id)
    caches = []
    for r in rows:
        rc = cache.requests.get(r.request_id)
        if rc is None:
            raise KeyError(f"request {r.request_id!r} is not live: admit it first")
        caches.append(rc)
    n_tokens = sum(lens)
    # everything below is whole-array work: a decode step has one token per row, and a Python
    # loop over rows would cost more than the kernels it feeds
    lens_np = np.asarray(lens, dtype=np.int64)
    row_pos0 = np.fromiter((rc.n_tokens for rc in caches), dtype=np.int32, count=n_rows)
    row_slot = np.fromiter((rc.slot for rc in caches), dtype=np.int32, count=n_rows)
    row_start = np.zeros(n_rows + 1, dtype=np.int32)
    np.cumsum(lens_np, out=row_start[1:])
    over = row_pos0.astype(np.int64) + lens_np > max_position
    if over.any():
        i = int(np.argmax(over))
        raise ValueError(f"request {rows[i].request_id!r}: position "
                         f"{int(row_pos0[i]) + lens[i] - 1} is beyond max_position "
                         f"{max_position}")
    if n_tokens == n_rows:
        flat = np.fromiter((r.tokens[0] for r in rows), dtype=np.int64, count=n_rows)
    else:
        flat = np.concatenate([np.asarray(r.tokens, dtype=np.int64) for r in rows])
    pending = [(i, r.pending) for i, r in enumerate(rows) if r.pending is not None]
    for i, j in pending:
        if lens[i] != 1 or j < 0:
            raise ValueError(f"request {rows[i].request_id!r}: a pending token is a row's only "
                             "token")
        flat[row_start[i]] = 0
    if flat.size and (flat.min() < 0 or flat.max() >= vocab_size):
        i = int(np.searchsorted(row_start[1:], int(np.argmax((flat < 0) | (flat >= vocab_size))),
                                side="right"))
        raise ValueError(f"request {rows[i].request_id!r}: token id out of range "
                         f"[0, {vocab_size})")
    token_ids = flat.astype(np.int32)
    for i, j in pending:
        token_ids[row_start[i]] = -1 - j
    token_row = np.repeat(np.arange(n_rows, dtype=np.int32), lens_np)
    positions = (np.arange(n_tokens, dtype=np.int32) - row_start[token_row] + row_pos0[token_row])
    logit_index: list[int] = []
    for i, row in enumerate(rows):
        if row.want:
            n, t = lens[i], int(row_start[i])
            for w in row.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {row.request_id!r}: wanted place {w} is not "
                                     f"among its {n} tokens")
                logit_index.append(t + w)
    tables = []
    for g in range(len(cache.groups)):
        arrays = [rc.tables_np[g][:len(rc.tables[g])] for rc in caches]
        width = max(a.size for a in arrays)
        if table_width is not None:
            if width > table_width:
                raise ValueError(f"a block table of {width} pages exceeds the fixed width "
                                 f"{table_width}")
            width = table_width
        tab = np.full((n_rows, max(width, 1)), -1, dtype=np.int32)
        for i, a in enumerate(arrays):
            tab[i, :a.size] = a
        tables.append(tab)
    li = np.asarray(logit_index, dtype=np.int32)
    single = [i for i, n in enumerate(lens) if n == 1]
    multi = [i for i, n in enumerate(lens) if n > 1]
    if pad:
        return _padded_batch(stager, pad_plan(n_tokens, len(single), len(multi), li.size),
                             token_ids, positions, token_row, row_start, row_pos0, row_slot, li,
                             single, multi, tables, lens)
    dev = stager.upload([token_ids, positions, token_row, row_start, row_pos0, row_slot, li,
                         np.asarray(single, dtype=np.int32), np.asarray(multi, dtype=np.int32),
                         *tables])
    single_np = np.asarray(single, dtype=np.int32)
    ctx_single = int(row_pos0[single_np].max()) + 1 if single else 0
    return StepBatch(
        n_tokens=n_tokens, n_rows=n_rows, n_out=len(logit_index), max_new=max(lens),
        max_context=int((row_pos0.astype(np.int64) + lens_np).max()),
        token_ids=dev[0], positions=dev[1], token_row=dev[2], row_start=dev[3],
        row_pos0=dev[4], row_slot=dev[5], logit_index=dev[6], single_rows=dev[7],
        multi_rows=dev[8], block_tables=dev[9:], n_single=len(single), n_multi=len(multi),
        max_new_multi=max((lens[i] for i in multi), default=0),
        max_context_single=ctx_single, context_bucket=context_bucket(ctx_single),
        wants_every_token=bool(li.size == n_tokens and (li == np.arange(n_tokens)).all()),
        host_row_new=lens, host_row_pos0=row_pos0.tolist(), n_real_tokens=n_tokens,
        n_real_out=len(logit_index))


def _padded_batch(stager: BatchStager, plan: PadPlan, token_ids, positions, token_row, row_start,
                  row_pos0, row_slot, li, single, multi, tables, lens) -> StepBatch:
    """The descriptor of a step at the sizes of ``plan``: see :class:`PadPlan`."""
    n_tokens, n_rows = int(token_ids.size), len(lens)
    rows_padded = plan.n_single + plan.n_multi + 1      # at least one row without tokens
    empty_row = rows_padded - 1

    def grown(a: np.ndarray, n: int, fill: int) -> np.ndarray:
        out = np.full(n, fill, dtype=np.int32)
        out[:a.size] = a
        return out

    single_np = np.asarray(single, dtype=np.int32)
    ctx_single = int(row_pos0[single_np].max()) + 1 if single else 0
    padded_tables = []
    for tab in tables:
        wide = np.full((rows_padded, tab.shape[1]), -1, dtype=np.int32)
        wide[:n_rows] = tab
        padded_tables.append(wide)
    dev = stager.upload([
        grown(token_ids, plan.n_tokens, 0), grown(positions, plan.n_tokens, 0),
        grown(token_row, plan.n_tokens, -1), grown(row_start, rows_padded + 1, n_tokens),
        grown(row_pos0, rows_padded, 0), grown(row_slot, rows_padded, 0),
        grown(li, plan.n_out, 0), grown(single_np, plan.n_single, empty_row),
        grown(np.asarray(multi, dtype=np.int32), plan.n_multi, empty_row), *padded_tables])
    return StepBatch(
        n_tokens=plan.n_tokens, n_rows=rows_padded, n_out=plan.n_out, max_new=plan.n_tokens,
        max_context=int((row_pos0.astype(np.int64) + np.asarray(lens, dtype=np.int64)).max()),
        token_ids=dev[0], positions=dev[1], token_row=dev[2], row_start=dev[3],
        row_pos0=dev[4], row_slot=dev[5], logit_index=dev[6], single_rows=dev[7],
        multi_rows=dev[8], block_tables=dev[9:], n_single=plan.n_single, n_multi=plan.n_multi,
        max_new_multi=plan.n_tokens if plan.n_multi else 0,
        max_context_single=ctx_single, context_bucket=context_bucket(ctx_single),
        host_row_new=list(lens) + [0] * (rows_padded - n_rows),
        host_row_pos0=row_pos0.tolist() + [0] * (rows_padded - n_rows),
        padded=True, n_real_tokens=n_tokens, n_real_out=int(li.size))
