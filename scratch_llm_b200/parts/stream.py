"""Handing a branch's output to the next norm without a kernel of its own, in decode steps.

In a pre-norm layer a branch ends with a matrix product whose output is added to the residual
stream, a norm follows, and the next branch starts with a matrix product
(src/scratch_llm/model.py:423-436 of the reference: ``x + Attn(Norm(x))``, ``x + FFN(Norm(x))``).
With a handful of tokens each of these is a short kernel and the step's time is the chain of
their starts and ends.  Two of the kernels can go, because an RMS norm's factor
``rsqrt(mean(x^2) + eps)`` is ONE number per token and commutes with the product that follows:

* the product that ends a branch (:class:`StreamSink`) adds its output into the 32-bit stream
  itself, writes ``stream * gain`` in the compute dtype as the next product's input, and leaves
  each token's sum of squares in shares (one per 8 features);
* the product that starts the next branch takes that input as it is (:class:`Normed`) and
  multiplies its outputs by the token's factor, which it gets by adding the shares in a fixed
  order.

The norm's arithmetic stays 32-bit with one rounding of the activations; only the place of
that rounding moves (before the factor instead of after it).  Parts opt in: a mixer or
feed-forward that can end with a sink takes a ``sink`` argument and says ``accepts_sink``; one
that can start from unfinished activations says so through ``accepts_normed(n_tokens)``; a norm
whose factor is one number per token says ``deferrable``.  Everything else runs as before.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops


@dataclass
class Normed:
    """Activations whose norm is not finished: the true value of row t is
    ``x[t] * rsqrt(shares[:, t].sum() / dim + eps)``."""

    x: torch.Tensor          # [tokens, dim] in the compute dtype: stream * gain
    shares: torch.Tensor     # float32 [parts, 8]: sums of squares of the stream, per token
    dim: int
    eps: float
    norm: object             # the norm this stands for

    @property
    def shape(self):
        return self.x.shape


class StreamSink:
    """Where a branch's last product may put its output: into ``resid``, prepared for ``norm``."""

    #: steps of more tokens never hand a norm over (the kernels that can are small-batch ones)
    MAX_TOKENS = 8

    def __init__(self, resid: torch.Tensor, norm) -> None:
        self.resid, self.norm = resid, norm

    def finish(self, linear, x: torch.Tensor):
        """``linear(x)`` added into the stream: a :class:`Normed` for the norm that follows, or,
        where the product's kernel cannot do that, the plain output (the norm then runs as
        usual)."""
        if not linear.can_sink(x):
            return linear(x)
        n, d = x.shape[0], linear.out_features
        x_out = torch.empty((n, d), dtype=x.dtype, device=x.device)
        shares = torch.empty((-(-d // 8), 8), dtype=torch.float32, device=x.device)
        ops.gemv_tma(x, linear.weight, None,
                     sink=(self.resid, self.norm.weight, x_out, shares))
        return Normed(x_out, shares, d, self.norm.eps, self.norm)
