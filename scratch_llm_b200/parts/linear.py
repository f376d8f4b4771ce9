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
#: from this many tokens on, gate/up + SwiGLU run on the fused tcgen05 kernel (measured at
#: 28672 x 4096: 99.5 against 104.9 us for the library product plus the activation kernel at 448
#: tokens, 179 against 204 us at 1,024; below it the 256-token tiles of an SM pair leave too many
#: of the 148 SMs idle: 97.8 against 80.0 us at 384)
FUSED_GEMM_MIN_TOKENS = 448


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
        # every CTA of the streaming kernel re-reads all activations, which costs as much as the
        # weights once the output is very wide and several tokens are in flight
        if self._persistent and x.shape[0] <= SMALL_BATCH and x.stride(0) % 8 == 0:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemv_tma(x, w, out)
        streams = x.shape[0] <= SMALL_BATCH and (x.shape[0] <= 2 or self.out_features <= 65536)
        if streams and self.in_features % 8 == 0 and x.stride(0) % 8 == 0:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemv_mma(x, w, out)
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())

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
        if fits and x.shape[0] >= FUSED_GEMM_MIN_TOKENS and half % 8 == 0:
            # tcgen05 kernel with the activation in its epilogue: the [tokens, 2F] intermediate
            # is never written
            return ops.gemm_tc(x, w, out, swiglu=True)
        return ops.swiglu(self(x), out)
