"""Position encodings.

``rotary``: cos and sin of ``position * theta^(-2j/head_dim)`` in a 32-bit table of
``max_position`` rows, built exactly as the reference builds its buffers
(src/scratch_llm/model.py:195-202); the rotation itself runs in the fused rotate-and-store
kernel in 32-bit.  ``interleaved`` True rotates the adjacent pairs (x[2j], x[2j+1]) as the
reference does (src/scratch_llm/model.py:204-220); False rotates (x[j], x[j + head_dim/2]),
the layout of checkpoints saved for the split-half rotation.

``none``: no position encoding (a mixer that needs none, or a test part).
"""

from __future__ import annotations

from typing import Mapping

import torch

from .base import BuildContext, PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    rotary_tables = True
    pad_safe = True   # a table lookup per token; padding tokens have position 0

    def __init__(self, head_dim: int, theta: float, max_position: int,
                 interleaved: bool = True) -> None:
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head size, got {head_dim}")
        self.head_dim, self.theta = head_dim, float(theta)
        self.max_position, self.interleaved = max_position, bool(interleaved)
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        """The reference's table, on the CPU in 32-bit."""
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2).float()
                                         / self.head_dim))
        freqs = torch.outer(torch.arange(self.max_position).float(), inv_freq)
        return freqs.cos(), freqs.sin()

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        cos, sin = self.tables()
        self.cos = cos.to(ctx.device).contiguous()
        self.sin = sin.to(ctx.device).contiguous()

    def apply(self, q, k, positions):  # the attention mixer uses the tables instead
        raise NotImplementedError("rotary positions are applied by the fused kernel")


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    pad_safe = True

    def __init__(self, **_: object) -> None:
        pass

    def apply(self, q, k, positions) -> None:
        return None
