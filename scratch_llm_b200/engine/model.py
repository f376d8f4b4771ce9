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
from ..parts.stream import Normed, StreamSink
from ..weights.loader import ParamSpec


def _spec_key(spec: PartSpec):
    return (spec.kind, tuple(sorted((k, repr(v)) for k, v in spec.args.items())))


#: kind of part (a value of a block's ``ROLES``) -> (registry, name used in error messages)
PART_KINDS = {"mixer": (MIXERS, "mixer"), "feed_forward": (FEED_FORWARDS, "feed-forward"),
              "norm": (NORMS, "norm"), "position": (POSITION_ENCODINGS, "position encoding")}


class _HeadEntry:
    """The output matrix as the part that follows the final norm: it can finish a norm handed
    over to it where its product can (see :mod:`scratch_llm_b200.parts.stream`)."""

    def __init__(self, model: "DecoderModel") -> None:
        self.model = model

    def accepts_normed(self, n_tokens: int) -> bool:
        head = self.model.lm_head
        return head is not None and head.takes_normed(n_tokens)


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.ctx: BuildContext | None = None
        positions: dict = {}
        self.blocks = []
        self._named_parts: list[tuple[str, object]] = []
        for layer in spec.layers:
            try:
                block_cls = BLOCKS[layer.block]
            except KeyError:
                raise ValueError(f"unknown block {layer.block!r}; registered: "
                                 f"{', '.join(sorted(BLOCKS))}") from None
            roles = dict(getattr(block_cls, "ROLES", {}))
            if set(roles) != set(layer.parts):
                raise ValueError(f"layer {layer.prefix!r}: block {layer.block!r} has the roles "
                                 f"{sorted(roles)}, the layer's spec gives {sorted(layer.parts)}")
            if sum(kind == "mixer" for kind in roles.values()) > 1:
                raise ValueError(f"block {layer.block!r} has several mixers: a layer has one "
                                 "cache entry, which one mixer owns")
            built = {}
            for role, kind in roles.items():
                part_spec = layer.parts[role]
                if kind not in PART_KINDS:
                    raise ValueError(f"block {layer.block!r}: role {role!r} has the unknown kind "
                                     f"{kind!r} (kinds: {', '.join(PART_KINDS)})")
                table, what = PART_KINDS[kind]
                if kind == "position":   # one table serves every layer that asks for the same
                    key = _spec_key(part_spec)
                    if key not in positions:
                        positions[key] = make(table, what, part_spec)
                    built[role] = positions[key]
                else:
                    built[role] = make(table, what, part_spec)
                    self._named_parts.append(
                        (f"{layer.prefix}.{layer.names.get(role, role)}", built[role]))
            block = block_cls(**built)
            block.parts = built          # role -> part, for whoever walks the model's parts
            block.cache_owner = next((built[r] for r, k in roles.items() if k == "mixer"), None)
            self.blocks.append(block)
        self._positions = list(positions.values())
        # per run: the (norm, part) the NEXT run's block starts with, for blocks that ask
        self._next_entry: list = []
        for i, run in enumerate(spec.order):
            block = self.blocks[run.layer]
            nxt = self.blocks[spec.order[i + 1].layer] if i + 1 < len(spec.order) else None
            entry = nxt.entry() if nxt is not None and hasattr(nxt, "entry") else None
            self._next_entry.append(entry if getattr(block, "takes_next_entry", False) else None)
        self.final_norm = make(NORMS, "norm", spec.final_norm)
        self._named_parts.append((spec.final_norm_name, self.final_norm))
        # what the first run starts with, for the embedding (if that block says, its norm's
        # factor is one number per token and its gain a vector `weight`)
        first = self.blocks[spec.order[0].layer] if spec.order else None
        entry = first.entry() if first is not None and hasattr(first, "entry") else None
        self._first_entry = entry if (entry is not None and getattr(entry[0], "deferrable", False)
                                      and hasattr(entry[1], "accepts_normed")) else None
        # the last run may prepare the final norm for the output matrix in steps that want the
        # logits of every token in order (decode steps), where no rows are gathered in between
        last = self.blocks[spec.order[-1].layer] if spec.order else None
        self._final_entry = ((self.final_norm, _HeadEntry(self))
                             if getattr(last, "takes_next_entry", False) else None)
        self.embedding: torch.Tensor | None = None
        self.lm_head: Linear | None = None

    def all_parts(self):
        """Every part of the model and every block, once (a position encoding that several
        layers share comes once)."""
        seen: dict[int, object] = {}
        for block in self.blocks:
            seen.setdefault(id(block), block)
            for part in block.parts.values():
                seen.setdefault(id(part), part)
        seen.setdefault(id(self.final_norm), self.final_norm)
        return list(seen.values())

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
                mixer = self.blocks[run.layer].cache_owner
                if mixer is not None:
                    kv[run.cache], st[run.cache] = mixer.kv_spec(), mixer.state_spec()
        return kv, st

    def head_dims(self) -> list[int]:
        return sorted({p.head_dim for p in self.all_parts()
                       if isinstance(getattr(p, "head_dim", None), int)})

    # --------------------------------------------------------------------------- forward

    def _embed(self, batch, resid: torch.Tensor):
        """The tokens' embeddings into the stream.  In steps of a few tokens the first run's
        norm is prepared for the product after it on the way (returned as what is pending),
        where that norm and that product can (scratch_llm_b200.parts.stream)."""
        s = self.spec
        n, d = batch.n_tokens, s.hidden_size
        entry = self._first_entry
        if (entry is not None and n <= StreamSink.MAX_TOKENS and d % 8 == 0
                and self.embedding.dtype == torch.bfloat16 and entry[1].accepts_normed(n)):
            norm = entry[0]
            x_out = torch.empty((n, d), dtype=torch.bfloat16, device=resid.device)
            shares = torch.empty((d // 8, 8), dtype=torch.float32, device=resid.device)
            ops.embed_prepare(batch.token_ids, self.embedding, resid, batch.pending_tokens,
                              s.embedding_multiplier, norm.weight, x_out, shares)
            return Normed(x_out, shares, d, norm.eps, norm)
        ops.embed(batch.token_ids, self.embedding, resid, batch.pending_tokens,
                  scale=s.embedding_multiplier)
        return None

    def forward(self, batch, cache) -> torch.Tensor | None:
        """Run the batch's tokens from the cache; returns logits [n_out, vocab] in 32-bit, or
        None when no logits are wanted."""
        s = self.spec
        resid = torch.empty((batch.n_tokens, s.hidden_size), dtype=torch.float32,
                            device=self.ctx.device)
        pending = self._embed(batch, resid)
        for i, run in enumerate(s.order):
            pages, group = cache.entry_pages(run.cache)
            view = CacheView(pages=pages,
                             block_table=batch.block_tables[group] if group is not None else None,
                             page_size=cache.page_size, state=cache.states[run.cache])
            block = self.blocks[run.layer]
            if i == len(s.order) - 1 and self._final_entry is not None and batch.wants_every_token:
                pending = block.forward(resid, pending, batch, view, run.write,
                                        next_entry=self._final_entry)
            elif self._next_entry[i] is not None:
                # what the next run starts with, so that this block's last product may prepare
                # it (the final norm works on gathered rows: nothing is prepared for it)
                pending = block.forward(resid, pending, batch, view, run.write,
                                        next_entry=self._next_entry[i])
            else:
                pending = block.forward(resid, pending, batch, view, run.write)
        if batch.n_out == 0:
            return None
        if isinstance(pending, Normed):      # prepared by the last run: every row, in order
            h = self.final_norm.forward(resid, pending)
        else:
            h = self.final_norm.forward(resid, pending, out_rows=batch.logit_index)
        logits = self.lm_head(h, out_dtype=torch.float32)
        if s.logit_scale != 1.0 or s.logit_softcap > 0:
            ops.logit_cap(logits, s.logit_scale, s.logit_softcap)
        return logits


def build_model(config) -> DecoderModel:
    """The model of a typed configuration, without weights and without touching a device."""
    from ..config import get_architecture

    arch = get_architecture(config.architecture)
    spec = config.model_spec()
    return arch.model_factory(spec) if arch.model_factory else DecoderModel(spec)
