"""Chooses the next token of every row that asked for logits, on the device.

Greedy rows take the argmax; the others draw from softmax(logits / temperature) after the
nucleus filter, each from its request's own counter-based generator: the draw for a request's
n-th token depends on (seed, n) only, so it is the same alone, in any batch, and after the
request was set back and recomputed.  Formulas: src/scratch_llm/sampling.py:60-95 of the
reference.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.bytes_read = 0   # device-to-host bytes so far
        self._argmax_scratch: dict[int, torch.Tensor] = {}

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               seeds: Sequence[int], counters: Sequence[int], want_logprobs: bool = False
               ) -> tuple[list[int], list[float] | None]:
        """One token per row of ``logits`` [n, vocab] (32-bit, on the device).  Returns host
        lists: the tokens and, if asked for, log_softmax(logits)[token] at temperature 1."""
        n = logits.shape[0]
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        lp = torch.empty(n, dtype=torch.float32, device=self.device) if want_logprobs else None
        if all(p.temperature == 0.0 for p in params) and lp is None:
            scratch = self._argmax_scratch.get(n)
            if scratch is None:   # one zero-filled scratch per batch size, kept
                scratch = torch.zeros(ops.argmax_scratch_bytes(n), dtype=torch.uint8,
                                      device=self.device)
                self._argmax_scratch[n] = scratch
            ops.argmax(logits, out, scratch, n)
        elif all(p.temperature == 0.0 for p in params):
            ops.sample(logits, out, logprob_out=lp)
        else:
            f = np.array([[p.temperature for p in params], [p.top_p for p in params]],
                         dtype=np.float32)
            i = np.array([[s & 0x7FFFFFFFFFFFFFFF for s in seeds], list(counters)], dtype=np.int64)
            fd = torch.from_numpy(f).to(self.device, non_blocking=True)
            idv = torch.from_numpy(i).to(self.device, non_blocking=True)
            ops.sample(logits, out, fd[0], fd[1], idv[0], idv[1], logprob_out=lp)
        tokens = out.tolist()  # the one device-to-host read of a step
        self.bytes_read += 4 * n * (2 if lp is not None else 1)
        return tokens, (lp.tolist() if lp is not None else None)
