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


class Linear:
    def __init__(self, weight: torch.Tensor) -> None:
        if weight.dim() != 2 or not weight.is_contiguous():
            raise ValueError("a Linear weight is a contiguous [out, in] matrix")
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        w = self.weight
        out_dtype = out_dtype or w.dtype
        if x.dtype != w.dtype:
            raise ValueError(f"Linear: input is {x.dtype}, weight is {w.dtype}")
        if w.dtype == torch.float32:
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32,
                              device=x.device)
            return ops.gemm_simt(x, w, out)
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())
