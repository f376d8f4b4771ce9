"""RMSNorm fused with the add of the pending residual delta.

``x * rsqrt(mean(x^2) + eps) * weight`` in 32-bit, eps inside the root, the weight after the
normalisation, one rounding at the end (src/scratch_llm/model.py:149-162 of the reference; its
eps is fixed at 1e-5 in code, here it is a parameter).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, Norm
from .registry import register_norm
from .stream import Normed


@register_norm("rmsnorm")
class RMSNorm(Norm):
    pad_safe = True   # every token by itself
    #: the norm's factor is one number per token: the product before it may prepare it and the
    #: product after it may apply it (scratch_llm_b200.parts.stream)
    deferrable = True

    def __init__(self, size: int, eps: float) -> None:
        self.size, self.eps = size, float(eps)
        self.weight: torch.Tensor | None = None
        self.dtype = torch.float32

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        self.weight = tensors["weight"].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.dtype = ctx.dtype

    def forward(self, resid: torch.Tensor, delta: torch.Tensor | None,
                out_rows: torch.Tensor | None = None):
        if isinstance(delta, Normed):
            # the product before this norm has already put its output into the stream and
            # prepared this norm: what is left is the tokens' factor, which the next product applies
            if delta.norm is not self or out_rows is not None:
                raise ValueError("a deferred norm reached a norm it was not prepared for")
            return delta
        n = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((n, self.size), dtype=self.dtype, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, out_rows)
