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
from .batch import BatchStager, RowInput, StepBatch, build_batch
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
    """A decode step of a fixed number of rows, captured as a CUDA graph."""

    def __init__(self, graph: torch.cuda.CUDAGraph, logits: torch.Tensor, pointers: tuple) -> None:
        self.graph, self.logits, self.pointers = graph, logits, pointers
        self.n_kernels = 0


class ModelRunner:
    """``cuda_graphs``: steps in which every row brings one token and wants its logits (decode)
    are captured once per (number of rows, context bucket) and replayed afterwards, in the manner of the
    reference's CudaGraphDecoder (src/scratch_llm/serving/cudagraph.py:31-96) and its
    per-batch-size buckets (src/scratch_llm/serving/graph_buckets.py:94-200): the descriptor
    arrays, the block tables (at their full width) and the pools keep their addresses, the
    kernels read contexts and pages on the device."""

    def __init__(self, model: DecoderModel, page_size: int, n_pages: int, max_requests: int,
                 cuda_graphs: bool = True) -> None:
        if model.ctx is None:
            raise ValueError("load the model's weights before building a runner")
        self.model = model
        self.device = model.ctx.device
        kv, st = model.cache_specs()
        self.cache = CacheManager(kv, st, page_size, n_pages, max_requests,
                                  dtype=model.ctx.dtype, device=self.device)
        self._stager = BatchStager(self.device)
        self.vocab_size = model.spec.vocab_size
        self.max_position = model.spec.max_position
        self.cuda_graphs = cuda_graphs and all(
            getattr(part, "capturable", True) for block in model.blocks
            for part in (block.mixer, block.feed_forward))
        self._table_width = self.cache.max_pages_per_request(self.max_position)
        self._captured: dict[tuple[int, int], _CapturedStep] = {}
        self.replayed_kernels = 0   # kernels of this package launched through graph replays
        self._seen_sizes: set[tuple[int, int]] = set()
        # tokens that a sampler chose and the host has not read yet: a row may name one of them
        # as its input (RowInput.pending), so that the next step can be launched before the
        # host has seen the tokens of this one
        self.pending_tokens = torch.zeros(max(1, max_requests), dtype=torch.int32,
                                          device=self.device)
        # room for the widest decode step, so that captured addresses stay valid
        self._stager.reserve(8 * (max_requests + 4) + 4 * max(1, len(self.cache.groups)) +
                             max_requests * (self._table_width + 4) * max(1, len(self.cache.groups)))

    # ----------------------------------------------------------------------- requests

    def admit(self, request_id: Hashable) -> bool:
        return self.cache.admit(request_id) is not None

    def release(self, request_id: Hashable) -> None:
        self.cache.release(request_id)

    def n_cached(self, request_id: Hashable) -> int:
        return self.cache.requests[request_id].n_tokens

    # --------------------------------------------------------------------------- step

    def build_batch(self, rows: Sequence[RowInput], table_width: int | None = None) -> StepBatch:
        for row in rows:
            if row.pending is not None and row.pending >= self.pending_tokens.numel():
                raise ValueError(f"request {row.request_id!r}: pending token {row.pending} is "
                                 f"beyond the buffer's {self.pending_tokens.numel()} entries")
        batch = build_batch(self.cache, self._stager, rows, self.vocab_size, self.max_position,
                            table_width=table_width)
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
            logits = self._decode_step(rows)
        else:
            logits = self.model.forward(self.build_batch(rows), self.cache)
        for row in rows:
            self.cache.commit(row.request_id, len(row.tokens))
        return logits

    def _decode_step(self, rows: Sequence[RowInput]) -> torch.Tensor:
        """Replay (or, at a size's second use, capture) the decode step for len(rows) rows."""
        n = len(rows)
        batch = self.build_batch(rows, table_width=self._table_width)
        pointers = (batch.token_ids.data_ptr(), batch.logit_index.data_ptr(),
                    tuple(t.data_ptr() for t in batch.block_tables))
        key = (n, batch.context_bucket)   # launch shapes depend on these two alone
        cap = self._captured.get(key)
        if cap is not None and cap.pointers == pointers:
            cap.graph.replay()
            self.replayed_kernels += cap.n_kernels
            return cap.logits.clone()   # the graph's own output is overwritten by the next replay
        if key not in self._seen_sizes:   # first use of this shape: run it plainly (warms up)
            self._seen_sizes.add(key)
            return self.model.forward(batch, self.cache)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        try:
            with torch.cuda.graph(graph):
                logits = self.model.forward(batch, self.cache)
        except RuntimeError:
            # a part that reads device values on the host while it runs cannot be captured:
            # from here on this runner launches every step plainly
            self.cuda_graphs = False
            self._captured.clear()
            torch.cuda.synchronize()
            return self.model.forward(batch, self.cache)
        cap = _CapturedStep(graph, logits, pointers)
        cap.n_kernels = ops.launch_count - before
        self._captured[key] = cap
        graph.replay()
        self.replayed_kernels += cap.n_kernels
        return logits.clone()


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
