"""Matrix products ``y = x @ W.T`` with the weight stored (out, in), without bias
(src/scratch_llm/model.py:125-133 of the reference).

32-bit path: the engine's own CUDA-core kernel with fused multiply-adds (true 32-bit; the
tensor cores' tf32 mode is never used).  bfloat16 path: the engine's tensor-core kernels where
they take the shape, else cuBLAS through ``torch.mm`` -- the reference's own model computes
every projection with the library product (``x @ self.weight.T``).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .stream import Normed


#: up to this many tokens the streaming small-batch kernel runs instead of the library product
SMALL_BATCH = 8
#: gate/up + SwiGLU run on the fused tcgen05 kernel (pairs of SMs, tiles of 256 tokens x 128
#: features, or x 112 where that needs no more rounds of tiles) from FUSED_GEMM_ALWAYS tokens on, and from FUSED_GEMM_MIN_TOKENS on where its tiles
#: fill the SM pairs' rounds to at least FUSED_GEMM_MIN_FILL (0.85) and the reduction is long enough to
#: carry a tile's start and end; else the library product plus the activation kernel.  Measured
#: inside graph replays, fused against library + activation, in us:
#:   28672 x 4096 (224 tiles up to 512 tokens: 3.03 rounds of 74 pairs, fill 0.76):
#:       448 tokens 112.8 / 110.7, 512: 119.3 / 109.2, 1,024: 215.7 / 227.5, 2,048: 370 / 427
#:   27648 x 5120 (216 tiles, 2.92 rounds, fill 0.97): 448: 114.6 / 120.5, 512: 124.8 / 132.9,
#:       1,024: 235.5 / 233.4, 2,048: 446 / 461
#:   16384 x 2048 (short reduction): 448: 37.5 / 32.6, 512: 35.8 / 32.4, 768: 46.9 / 46.3,
#:       1,024: 61.8 / 62.8, 2,048: 105 / 142
FUSED_GEMM_MIN_TOKENS = 448
FUSED_GEMM_ALWAYS = 1024
FUSED_GEMM_MIN_FILL = 0.85
FUSED_GEMM_MIN_K = 4096


class Linear:
    def __init__(self, weight: torch.Tensor) -> None:
        if weight.dim() != 2 or not weight.is_contiguous():
            raise ValueError("a Linear weight is a contiguous [out, in] matrix")
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        # the persistent small-batch kernel takes this matrix (plain and as [gate; up]): its
        # workspace is made now, so that no step allocates it
        self._persistent = self._persistent_swiglu = False
        if weight.dtype == torch.bfloat16 and weight.is_cuda:
            n, k = self.out_features, self.in_features
            self._persistent = ops.gemv_tma_supports(1, n, k, False)
            self._persistent_swiglu = n % 2 == 0 and ops.gemv_tma_supports(1, n, k, True)
            if self._persistent or self._persistent_swiglu:
                ops.gemv_tma_reserve(n, k, False, weight.device)

    def takes_normed(self, n_tokens: int, swiglu: bool = False) -> bool:
        """Whether this product can start from activations whose norm is not finished
        (:class:`~scratch_llm_b200.parts.stream.Normed`): the persistent small-batch kernel
        applies the tokens' factors to its outputs."""
        return n_tokens <= SMALL_BATCH and (self._persistent_swiglu if swiglu
                                            else self._persistent)

    def can_sink(self, x: torch.Tensor) -> bool:
        """Whether this product can add its output into the residual stream itself."""
        return (self._persistent and isinstance(x, torch.Tensor) and x.shape[0] <= SMALL_BATCH
                and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0)

    def __call__(self, x, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        w = self.weight
        out_dtype = out_dtype or w.dtype
        if isinstance(x, Normed):
            if not self.takes_normed(x.x.shape[0]):
                raise ValueError("this product cannot finish a deferred norm (the part that "
                                 "handed it over must ask takes_normed first)")
            out = torch.empty((x.x.shape[0], self.out_features), dtype=out_dtype,
                              device=x.x.device)
            return ops.gemv_tma(x.x, w, out, scale=(x.shares, x.dim, x.eps))
        if x.dtype != w.dtype:
            raise ValueError(f"Linear: input is {x.dtype}, weight is {w.dtype}")
        if w.dtype == torch.float32:
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32,
                              device=x.device)
            return ops.gemm_simt(x, w, out)
        if self._persistent and x.shape[0] <= SMALL_BATCH and x.stride(0) % 8 == 0:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemv_tma(x, w, out)
        # shapes the persistent kernel does not take: every CTA of the older streaming kernel
        # re-reads all activations, which costs as much as the weights once the output is very
        # wide and several tokens are in flight
        streams = x.shape[0] <= SMALL_BATCH and (x.shape[0] <= 2 or self.out_features <= 65536)
        if streams and self.in_features % 8 == 0 and x.stride(0) % 8 == 0:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemv_mma(x, w, out)
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())

    def _fused_pays(self, m: int, half: int) -> bool:
        """Whether gate/up + SwiGLU of ``m`` tokens is faster on the fused tcgen05 kernel than
        as library product + activation kernel (see FUSED_GEMM_MIN_TOKENS)."""
        if m >= FUSED_GEMM_ALWAYS:
            return True
        if m < FUSED_GEMM_MIN_TOKENS or self.in_features < FUSED_GEMM_MIN_K:
            return False
        pairs = max(1, ops.sm_count(self.weight.device) // 2)
        tiles = -(-m // 256) * -(-half // 128)
        return tiles / (-(-tiles // pairs) * pairs) >= FUSED_GEMM_MIN_FILL

    def swiglu(self, x: torch.Tensor) -> torch.Tensor:
        """For a weight [gate rows; up rows]: silu(x gate^T) * (x up^T), fused where a kernel
        takes the shape."""
        w = self.weight
        half = self.out_features // 2
        if isinstance(x, Normed):
            if not self.takes_normed(x.x.shape[0], swiglu=True):
                raise ValueError("this product cannot finish a deferred norm (the part that "
                                 "handed it over must ask takes_normed first)")
            out = torch.empty((x.x.shape[0], half), dtype=x.x.dtype, device=x.x.device)
            return ops.gemv_tma(x.x, w, out, swiglu=True, scale=(x.shares, x.dim, x.eps))
        out = torch.empty((x.shape[0], half), dtype=x.dtype, device=x.device)
        fits = (w.dtype == torch.bfloat16 and self.in_features % 8 == 0
                and x.stride(0) % 8 == 0)
        if fits and x.shape[0] <= SMALL_BATCH:
            if self._persistent_swiglu:
                return ops.gemv_tma(x, w, out, swiglu=True)
            return ops.gemv_mma(x, w, out, swiglu=True)
        if fits and half % 8 == 0 and self._fused_pays(x.shape[0], half):
            # tcgen05 kernel with the activation in its epilogue: the [tokens, 2F] intermediate
            # is never written
            return ops.gemm_tc(x, w, out, swiglu=True)
        return ops.swiglu(self(x), out)
