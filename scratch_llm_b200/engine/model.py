"""The generic decoder: embedding, the layers of a :class:`ModelSpec` in its run order, final
norm, output matrix on the wanted rows only.

embed -> blocks -> final norm -> output matrix is src/scratch_llm/model.py:471-505 of the
reference, which computes logits at every position (:480) and lets callers slice the last one
(src/scratch_llm/serving/continuous.py:496-498); here only the rows named by
``batch.logit_index`` pass through the final norm and the output matrix.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import ModelSpec, PartSpec
from ..kernels import ops
from ..parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, BuildContext,
                     CacheView, KVSpec, StateSpec, make)
from ..parts.linear import Linear
from ..weights.loader import ParamSpec


def _spec_key(spec: PartSpec):
    return (spec.kind, tuple(sorted((k, repr(v)) for k, v in spec.args.items())))


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.ctx: BuildContext | None = None
        positions: dict = {}
        self.blocks = []
        self._named_parts: list[tuple[str, object]] = []
        for layer in spec.layers:
            key = _spec_key(layer.position)
            if key not in positions:  # one table serves every layer that asks for the same
                positions[key] = make(POSITION_ENCODINGS, "position encoding", layer.position)
            mixer = make(MIXERS, "mixer", layer.mixer)
            ff = make(FEED_FORWARDS, "feed-forward", layer.feed_forward)
            n1 = make(NORMS, "norm", layer.mixer_norm)
            n2 = make(NORMS, "norm", layer.feed_forward_norm)
            try:
                block_cls = BLOCKS[layer.block]
            except KeyError:
                raise ValueError(f"unknown block {layer.block!r}; registered: "
                                 f"{', '.join(sorted(BLOCKS))}") from None
            self.blocks.append(block_cls(mixer, ff, n1, n2, positions[key]))
            for role, part in (("mixer", mixer), ("feed_forward", ff), ("mixer_norm", n1),
                               ("feed_forward_norm", n2)):
                self._named_parts.append((f"{layer.prefix}.{layer.names.get(role, role)}", part))
        self._positions = list(positions.values())
        self.final_norm = make(NORMS, "norm", spec.final_norm)
        self._named_parts.append((spec.final_norm_name, self.final_norm))
        self.embedding: torch.Tensor | None = None
        self.lm_head: Linear | None = None

    # --------------------------------------------------------------------------- weights

    def param_specs(self) -> dict[str, ParamSpec]:
        s = self.spec
        specs = {s.embed_name: ParamSpec((s.vocab_size, s.hidden_size))}
        for prefix, part in self._named_parts:
            for name, p in part.param_specs().items():
                specs[f"{prefix}.{name}"] = p
        if not s.tie_embeddings:
            specs[s.lm_head_name] = ParamSpec((s.vocab_size, s.hidden_size))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        s = self.spec
        self.ctx = ctx
        for prefix, part in self._named_parts:
            mine = {name: tensors[f"{prefix}.{name}"] for name in part.param_specs()}
            part.load(mine, ctx)
        for pos in self._positions:
            pos.load({}, ctx)
        self.embedding = tensors[s.embed_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()
        head = self.embedding if s.tie_embeddings else \
            tensors[s.lm_head_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()
        self.lm_head = Linear(head)

    # ----------------------------------------------------------------------------- cache

    def cache_specs(self) -> tuple[list[KVSpec | None], list[StateSpec | None]]:
        """What each cache entry needs: the spec of the run that writes it."""
        n = self.spec.n_cache_entries
        ids = sorted({r.cache for r in self.spec.order})
        if ids != list(range(n)):
            raise ValueError(f"cache entries must be numbered 0..{n - 1}, got {ids}")
        kv: list[KVSpec | None] = [None] * n
        st: list[StateSpec | None] = [None] * n
        for run in self.spec.order:
            if run.write:
                mixer = self.blocks[run.layer].mixer
                kv[run.cache], st[run.cache] = mixer.kv_spec(), mixer.state_spec()
        return kv, st

    def head_dims(self) -> list[int]:
        return sorted({b.mixer.head_dim for b in self.blocks if hasattr(b.mixer, "head_dim")})

    # --------------------------------------------------------------------------- forward

    def forward(self, batch, cache) -> torch.Tensor | None:
        """Run the batch's tokens from the cache; returns logits [n_out, vocab] in 32-bit, or
        None when no logits are wanted."""
        s = self.spec
        resid = torch.empty((batch.n_tokens, s.hidden_size), dtype=torch.float32,
                            device=self.ctx.device)
        ops.embed(batch.token_ids, self.embedding, resid, batch.pending_tokens)
        pending = None
        for run in s.order:
            pages, group = cache.entry_pages(run.cache)
            view = CacheView(pages=pages,
                             block_table=batch.block_tables[group] if group is not None else None,
                             page_size=cache.page_size, state=cache.states[run.cache])
            pending = self.blocks[run.layer].forward(resid, pending, batch, view, run.write)
        if batch.n_out == 0:
            return None
        h = self.final_norm.forward(resid, pending, out_rows=batch.logit_index)
        return self.lm_head(h, out_dtype=torch.float32)


def build_model(config) -> DecoderModel:
    """The model of a typed configuration, without weights and without touching a device."""
    from ..config import get_architecture

    arch = get_architecture(config.architecture)
    spec = config.model_spec()
    return arch.model_factory(spec) if arch.model_factory else DecoderModel(spec)
