"""Dense SwiGLU feed-forward: ``W_down( silu(W_gate x) * (W_up x) )`` without biases
(src/scratch_llm/model.py:223-237 of the reference; its w1 is the gate, w3 the up and w2 the
down matrix).  Gate and up are fused into one [2F, d] matrix at load.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..weights.loader import ParamSpec
from .base import BuildContext, FeedForward
from .linear import Linear
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    pad_safe = True   # every token by itself
    accepts_sink = True   # forward() takes sink=: the down projection may feed the stream itself

    def accepts_normed(self, n_tokens: int) -> bool:
        return self.gate_up is not None and self.gate_up.takes_normed(n_tokens, swiglu=True)

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names: Mapping[str, str] | None = None) -> None:
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight",
                      "down": "down_proj.weight", **(names or {})}
        self.gate_up: Linear | None = None
        self.down: Linear | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        d, f = self.hidden_size, self.intermediate_size
        return {self.names["gate"]: ParamSpec((f, d)), self.names["up"]: ParamSpec((f, d)),
                self.names["down"]: ParamSpec((d, f))}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        self.gate_up = Linear(torch.cat([put(tensors[self.names["gate"]]),
                                         put(tensors[self.names["up"]])], 0).contiguous())
        self.down = Linear(put(tensors[self.names["down"]]).contiguous())

    def forward(self, x, sink=None):
        y = self.gate_up.swiglu(x)
        return self.down(y) if sink is None else sink.finish(self.down, y)
