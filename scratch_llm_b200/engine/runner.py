"""The step function: one batch of (request, its next tokens) through the model, from the
cache, returning the logits at the wanted places.

The reference has no single step function: admission prefills and lockstep decodes are
separate forwards (src/scratch_llm/serving/continuous.py:284-398) and a mixed batch is left
unbuilt (bench/RESULTS.md:340-350).  Here the scheduler, the Python entry point and
``bin/trace_run`` all drive :meth:`ModelRunner.step`.
"""

from __future__ import annotations

from pathlib import Path
from typing import Hashable, Sequence

import torch

from ..cache import CacheManager
from ..config import load_config
from ..kernels import ops
from ..parts import BuildContext
from ..weights import load_tensors
from .batch import PAD_MAX_TOKENS, BatchStager, RowInput, StepBatch, build_batch
from .model import DecoderModel, build_model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32}


class OutOfPages(RuntimeError):
    """A step was asked to store tokens for which the cache has no free pages."""


def require_cuda() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("scratch_llm_b200 runs on a CUDA device (sm_100a) only: there is no "
                           "CPU path")
    return torch.device("cuda", torch.cuda.current_device())


class _CapturedStep:
    """A step of fixed launch shapes, captured as a CUDA graph."""

    def __init__(self, graph: torch.cuda.CUDAGraph, logits: torch.Tensor | None,
                 pointers: tuple) -> None:
        self.graph, self.logits, self.pointers = graph, logits, pointers
        self.n_kernels = 0


#: decode steps of more rows than this are padded to the next multiple of 8 rows (below, a
#: step's few rows choose how many CTAs share a row's keys, and padding would spoil the choice)
DECODE_EXACT_ROWS = 8
#: a step that wants more logits than this is not padded and captured: a captured step keeps
#: its output [wanted, vocabulary] in 32-bit allocated
PAD_MAX_WANTED = 64
#: captured graphs a runner keeps; the one used longest ago goes first
MAX_CAPTURED_STEPS = 192
#: a decode shape is captured at its second use: every later step has it again (capturing at
#: the first use costs more than a plain step and a capture after it, 28 against 10 + 11 ms at
#: Llama-3-8B sizes: what a first use sets up is cheaper outside a capture).  A padded
#: shape is captured once it has come this often: a capture costs as much as the launches of
#: some ten plain steps and saves a tenth of a step each time, and many shapes come only a few times
CAPTURE_PADDED_AFTER = 24


class ModelRunner:
    """``cuda_graphs``: steps in which every row brings one token and wants its logits (decode)
    are captured once per (number of rows, context bucket) and replayed afterwards, in the manner of the
    reference's CudaGraphDecoder (src/scratch_llm/serving/cudagraph.py:31-96) and its
    per-batch-size buckets (src/scratch_llm/serving/graph_buckets.py:94-200): the descriptor
    arrays, the block tables (at their full width) and the pools keep their addresses, the
    kernels read contexts and pages on the device.  Other steps of up to PAD_MAX_TOKENS tokens
    (portions of prompts, alone or beside decoded tokens) are padded to a few sizes
    (engine/batch.py::pad_plan) and captured per padded shape, if every part of the model
    is ``pad_safe``: launched plainly, such a step costs the host more than the device.
    ``poison_free_pages``: a debugging aid of the cache manager (free pages hold NaN)."""

    def __init__(self, model: DecoderModel, page_size: int, n_pages: int, max_requests: int,
                 cuda_graphs: bool = True, poison_free_pages: bool = False) -> None:
        if model.ctx is None:
            raise ValueError("load the model's weights before building a runner")
        self.model = model
        self.device = model.ctx.device
        kv, st = model.cache_specs()
        self.cache = CacheManager(kv, st, page_size, n_pages, max_requests,
                                  dtype=model.ctx.dtype, device=self.device,
                                  poison_free_pages=poison_free_pages)
        self._stager = BatchStager(self.device)
        self.vocab_size = model.spec.vocab_size
        self.max_position = model.spec.max_position
        # every part of every layer has a say (mixers, feed-forwards, norms, position
        # encodings, the blocks themselves, the final norm), with the same defaults
        self.cuda_graphs = cuda_graphs and all(
            getattr(part, "capturable", True) for part in model.all_parts())
        self.pad_small_steps = self.cuda_graphs and all(
            getattr(part, "pad_safe", False) for part in model.all_parts())
        self._table_width = self.cache.max_pages_per_request(self.max_position)
        self._captured: dict[tuple, _CapturedStep] = {}
        self._graph_pool = None     # memory shared by the captured steps (they never overlap)
        self.replayed_kernels = 0   # kernels of this package launched through graph replays
        self.replayed_steps = 0
        self._uses: dict[tuple, int] = {}   # how often an uncaptured shape has come
        self.capture_padded_after = CAPTURE_PADDED_AFTER
        self._capture_stream: torch.cuda.Stream | None = None
        # tokens that a sampler chose and the host has not read yet: a row may name one of them
        # as its input (RowInput.pending), so that the next step can be launched before the
        # host has seen the tokens of this one
        self.pending_tokens = torch.zeros(max(1, max_requests), dtype=torch.int32,
                                          device=self.device)
        # room for the widest decode step, so that captured addresses stay valid
        groups = max(1, len(self.cache.groups))
        # a padded step has up to 7 single rows, one empty row and as many multi rows more
        rows = 2 * max_requests + 16
        self._stager.reserve(3 * (PAD_MAX_TOKENS + 64) + 8 * (rows + 4) + 4 * groups +
                             rows * (self._table_width + 4) * groups)

    # ----------------------------------------------------------------------- requests

    def admit(self, request_id: Hashable) -> bool:
        return self.cache.admit(request_id) is not None

    def release(self, request_id: Hashable) -> None:
        self.cache.release(request_id)

    def n_cached(self, request_id: Hashable) -> int:
        return self.cache.requests[request_id].n_tokens

    # --------------------------------------------------------------------------- step

    def build_batch(self, rows: Sequence[RowInput], table_width: int | None = None,
                    pad: bool = False) -> StepBatch:
        for row in rows:
            if row.pending is not None and row.pending >= self.pending_tokens.numel():
                raise ValueError(f"request {row.request_id!r}: pending token {row.pending} is "
                                 f"beyond the buffer's {self.pending_tokens.numel()} entries")
        batch = build_batch(self.cache, self._stager, rows, self.vocab_size, self.max_position,
                            table_width=table_width, pad=pad)
        batch.pending_tokens = self.pending_tokens
        return batch

    def step(self, rows: Sequence[RowInput]) -> torch.Tensor | None:
        """Run exactly the tokens of ``rows`` as one batch from the cache that earlier steps
        left; store their keys and values; return logits [wanted, vocab] in 32-bit in the
        order of the rows and of each row's ``want`` (None if nothing is wanted)."""
        if not rows:
            return None
        for row in rows:
            if row.request_id not in self.cache.requests:
                raise KeyError(f"request {row.request_id!r} is not live: admit it first")
            if not self.cache.reserve(row.request_id, len(row.tokens)):
                raise OutOfPages(f"no free pages for {len(row.tokens)} more tokens of request "
                                 f"{row.request_id!r} (free per group: {self.cache.free_pages()})")
        if self.cuda_graphs and all(len(r.tokens) == 1 and len(r.want) == 1 for r in rows):
            # up to DECODE_EXACT_ROWS rows a decode step is captured as it is; above, for the
            # next multiple of 8 rows, so that requests that end one by one do not ask for a
            # capture each
            pad = self.pad_small_steps and len(rows) > DECODE_EXACT_ROWS
            batch = self.build_batch(rows, table_width=self._table_width, pad=pad)
            # launch shapes depend on these two alone
            logits = self._graph_step(batch, (batch.n_tokens, batch.context_bucket), 2)
            if pad and batch.n_real_out != batch.n_out:
                logits = logits[:batch.n_real_out]
        elif (self.pad_small_steps and sum(len(r.tokens) for r in rows) <= PAD_MAX_TOKENS
              and sum(len(r.want) for r in rows) <= PAD_MAX_WANTED):
            # block tables as wide as the longest row needs, rounded up to a power of two
            # (at their full width a model with very long positions would upload megabytes)
            pages = max(-(-(self.cache.requests[r.request_id].n_tokens + len(r.tokens))
                          // self.cache.page_size) for r in rows)
            width = 8
            while width < pages:
                width *= 2
            width = min(width, self._table_width)
            batch = self.build_batch(rows, table_width=width, pad=True)
            logits = self._graph_step(batch, ("padded", batch.n_tokens, batch.n_single,
                                              batch.n_multi, batch.n_out, batch.context_bucket,
                                              width), self.capture_padded_after)
            if logits is not None and batch.n_real_out != batch.n_out:
                logits = logits[:batch.n_real_out]
        else:
            logits = self.model.forward(self.build_batch(rows), self.cache)
        for row in rows:
            self.cache.commit(row.request_id, len(row.tokens))
        return logits

    def _graph_step(self, batch: StepBatch, key: tuple, capture_at: int) -> torch.Tensor | None:
        """Replay the step captured for ``key`` (the launch shapes of the batch); capture it
        at the key's use number ``capture_at``, run it plainly before."""
        pointers = (batch.token_ids.data_ptr(), batch.logit_index.data_ptr(),
                    tuple(t.data_ptr() for t in batch.block_tables))
        cap = self._captured.get(key)
        if cap is not None and cap.pointers == pointers:
            self._captured[key] = self._captured.pop(key)   # most recently used last
            cap.graph.replay()
            self.replayed_kernels += cap.n_kernels
            self.replayed_steps += 1
            # the graph's own output is overwritten by the next replay
            return None if cap.logits is None else cap.logits.clone()
        uses = self._uses.get(key, 0) + 1
        if uses < capture_at:   # (the first use also warms up what the capture must not do)
            self._uses[key] = uses
            return self.model.forward(batch, self.cache)
        self._uses.pop(key, None)
        cap = self._capture(batch, pointers)
        if cap is None:
            return self.model.forward(batch, self.cache)
        self._captured.pop(key, None)
        self._captured[key] = cap
        while len(self._captured) > MAX_CAPTURED_STEPS:
            self._captured.pop(next(iter(self._captured)))
        cap.graph.replay()
        self.replayed_kernels += cap.n_kernels
        self.replayed_steps += 1
        return None if cap.logits is None else cap.logits.clone()

    def _capture(self, batch: StepBatch, pointers: tuple) -> _CapturedStep | None:
        """Record the step into a graph on a side stream.  All graphs share one memory pool
        (they are replayed one after the other on one stream; their outputs stay allocated).
        Unlike ``torch.cuda.graph`` this neither collects garbage nor empties the allocator's
        cache, which cost more than the capture itself."""
        if self._graph_pool is None or not self._captured:
            # (a pool lives as long as a graph uses it: with none left, a new one is needed)
            self._graph_pool = torch.cuda.graph_pool_handle()
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        stream = self._capture_stream
        stream.wait_stream(torch.cuda.current_stream())
        failed = False
        with torch.cuda.stream(stream):
            graph.capture_begin(pool=self._graph_pool)
            try:
                logits = self.model.forward(batch, self.cache)
            except RuntimeError:
                failed = True
            try:
                graph.capture_end()
            except RuntimeError:
                failed = True
        torch.cuda.current_stream().wait_stream(stream)
        if failed:
            # a part that reads device values on the host while it runs cannot be captured:
            # from here on this runner launches every step plainly
            self.cuda_graphs = self.pad_small_steps = False
            self._captured.clear()
            torch.cuda.synchronize()
            return None
        cap = _CapturedStep(graph, logits, pointers)
        cap.n_kernels = ops.launch_count - before
        return cap


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
               device: torch.device | None = None, verbose: bool = True) -> DecoderModel:
    """Open a model folder: the class comes from config.json's architecture, the tensors from
    model.safetensors by name."""
    device = device or require_cuda()
    dt = DTYPES[dtype] if isinstance(dtype, str) else dtype
    config = load_config(model_dir)
    model = build_model(config)
    ops.prepare(model.head_dims(), verbose=verbose)
    aliases = config.reference_aliases() if hasattr(config, "reference_aliases") else None
    optional = {model.spec.lm_head_name: model.spec.embed_name} if model.spec.tie_embeddings \
        else None
    tensors = load_tensors(model_dir, model.param_specs(), aliases, optional)
    model.load(tensors, BuildContext(dtype=dt, device=device))
    model.config = config
    return model
