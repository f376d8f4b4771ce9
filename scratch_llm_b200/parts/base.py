"""Interfaces of the parts a layer is put together from.

A part is built from explicit sizes and constants (never from a model's configuration
object), states which tensors it wants (:meth:`Part.param_specs`, names relative to its own
prefix), receives them once (:meth:`Part.load`) and is then called by a block inside the step
function.  No part knows which model it is in.

=================  ==========================================================================
part               call
=================  ==========================================================================
Norm               ``forward(resid, delta, out_rows=None) -> normed``: add the pending
                   ``delta`` into the 32-bit residual stream, return norm(resid) in the compute
                   dtype; with ``out_rows`` only those rows are normed and resid is not written
PositionEncoding   ``apply(q, k, positions)`` in place on [N, heads, head_dim] views, or, for
                   the rotary encoding, its tables handed to the fused rotate-and-store kernel
Mixer              ``forward(x, batch, cache, write, position) -> [N, hidden]``; states what it
                   caches through ``kv_spec()`` (paged keys and values) and ``state_spec()``
                   (fixed-size state per request)
FeedForward        ``forward(x) -> [N, hidden]``
Block              ``forward(resid, pending, batch, cache, write) -> pending``: the arrangement
                   of a layer's parts around the residual stream; its ``ROLES`` says which
                   parts it has (role -> kind of part), and it is built with one keyword
                   argument per role
=================  ==========================================================================
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Mapping

import torch

from ..weights.loader import ParamSpec

if TYPE_CHECKING:
    from ..engine.batch import StepBatch


@dataclass(frozen=True)
class BuildContext:
    """Where and in which precision a model is built.  ``dtype`` is the dtype of matrix-product
    operands and of the cache: ``torch.bfloat16`` (serving) or ``torch.float32`` (everything in
    true 32-bit)."""

    dtype: torch.dtype
    device: torch.device


@dataclass(frozen=True)
class KVSpec:
    """Paged keys and values one cache entry needs per token.  ``window`` None keeps every key;
    a number keeps the last ``window`` keys and lets older pages be given back."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size that one cache entry keeps per live request."""

    shape: tuple[int, ...]
    dtype: torch.dtype


@dataclass
class CacheView:
    """What one run of a layer sees of the cache in this step."""

    pages: torch.Tensor | None = None        # [n_pages, 2, n_kv_heads, page_size, head_dim]
    block_table: torch.Tensor | None = None  # int32 [rows, max_pages]; -1 where no page is held
    page_size: int = 0
    state: torch.Tensor | None = None        # [n_slots, *StateSpec.shape]


class Part:
    #: False if ``forward`` reads device values on the host (``.item()``, ``.tolist()``) or
    #: otherwise cannot be recorded into a CUDA graph; decode steps are then launched plainly
    capturable = True
    #: True if the part takes a padded step: tokens after the last row's that belong to no row
    #: (``token_row`` -1, id 0, position 0; their activations are never read), rows without
    #: tokens, and counts in the batch that include them.  Small steps of any shape are then
    #: padded to a few sizes and replayed as CUDA graphs.  Parts that work on every token by
    #: itself are safe; the default is the careful one.
    pad_safe = False

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        """Take the part's tensors (CPU or device, as stored) onto the device in the dtype the
        part computes in."""


class Norm(Part):
    def forward(self, resid: torch.Tensor, delta: torch.Tensor | None,
                out_rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    #: True if the attention mixer may hand cos/sin tables to its fused rotate-and-store kernel
    rotary_tables = False

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def kv_spec(self) -> KVSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, batch: "StepBatch", cache: CacheView, write: bool,
                position: PositionEncoding) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of a layer's parts.  ``ROLES`` maps each role the arrangement has onto
    the kind of part that fills it: ``"mixer"``, ``"feed_forward"``, ``"norm"`` or
    ``"position"`` (the registry the part's spec is looked up in).  The model builds the parts
    from the layer's specs and constructs the block with one keyword argument per role.  At most
    one role may be a mixer: it owns the layer's cache entry."""

    ROLES: dict[str, str] = {}
    capturable = True
    pad_safe = False
    #: True if forward() takes ``next_entry=``: the (norm, part) that the next block in the run
    #: order starts with (None at the end), so that the block's last product may prepare it
    takes_next_entry = False

    def entry(self):
        """(norm, part) this block starts with, for the block before it; None: not said."""
        return None

    def forward(self, resid: torch.Tensor, pending: torch.Tensor | None, batch: "StepBatch",
                cache: CacheView, write: bool) -> torch.Tensor:
        raise NotImplementedError
