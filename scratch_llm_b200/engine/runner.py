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


class ModelRunner:
    def __init__(self, model: DecoderModel, page_size: int, n_pages: int, max_requests: int
                 ) -> None:
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

    # ----------------------------------------------------------------------- requests

    def admit(self, request_id: Hashable) -> bool:
        return self.cache.admit(request_id) is not None

    def release(self, request_id: Hashable) -> None:
        self.cache.release(request_id)

    def n_cached(self, request_id: Hashable) -> int:
        return self.cache.requests[request_id].n_tokens

    # --------------------------------------------------------------------------- step

    def build_batch(self, rows: Sequence[RowInput]) -> StepBatch:
        return build_batch(self.cache, self._stager, rows, self.vocab_size, self.max_position)

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
        batch = self.build_batch(rows)
        logits = self.model.forward(batch, self.cache)
        for row in rows:
            self.cache.commit(row.request_id, len(row.tokens))
        return logits


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
