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


class PendingSample:
    """Tokens that were chosen on the device and are on their way to the host."""

    def __init__(self, n: int, host_tokens: torch.Tensor, host_lp: torch.Tensor | None,
                 event: torch.cuda.Event) -> None:
        self._n, self._tokens, self._lp, self._event = n, host_tokens, host_lp, event

    def result(self) -> tuple[list[int], list[float] | None]:
        """Waits for the copy and returns host lists: the tokens and, if they were asked for,
        their log-probabilities."""
        self._event.synchronize()
        tokens = self._tokens[:self._n].tolist()
        return tokens, (self._lp[:self._n].tolist() if self._lp is not None else None)


class Sampler:
    #: pinned host buffers that take turns; at most this many samples may be in flight
    IN_FLIGHT = 4

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.bytes_read = 0   # device-to-host bytes so far
        self._argmax_scratch: dict[int, torch.Tensor] = {}
        self._host: list[tuple[torch.Tensor, torch.Tensor, torch.cuda.Event]] = []
        self._turn = 0

    def _host_buffers(self, n: int) -> tuple[torch.Tensor, torch.Tensor, torch.cuda.Event]:
        if not self._host or self._host[0][0].numel() < n:
            size = max(64, 1 << (n - 1).bit_length())
            self._host = [(torch.empty(size, dtype=torch.int32, pin_memory=True),
                           torch.empty(size, dtype=torch.float32, pin_memory=True),
                           torch.cuda.Event()) for _ in range(self.IN_FLIGHT)]
        self._turn = (self._turn + 1) % self.IN_FLIGHT
        return self._host[self._turn]

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               seeds: Sequence[int], counters: Sequence[int], want_logprobs: bool = False
               ) -> tuple[list[int], list[float] | None]:
        """One token per row of ``logits`` [n, vocab] (32-bit, on the device).  Returns host
        lists: the tokens and, if asked for, log_softmax(logits)[token] at temperature 1."""
        return self.sample_async(logits, params, seeds, counters, want_logprobs).result()

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     seeds: Sequence[int], counters: Sequence[int], want_logprobs: bool = False,
                     out: torch.Tensor | None = None) -> PendingSample:
        """Like :meth:`sample`, but returns at once: the tokens are written to ``out`` (int32
        [n] on the device, if given) and copied to pinned host memory behind the kernels;
        ``result()`` of the returned object waits for that copy (the one device-to-host read
        of a step)."""
        n = logits.shape[0]
        if out is None:
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
            # (no top_p below 1: the kernel is told so, and need not look for a nucleus)
            nucleus = fd[1] if any(p.top_p < 1.0 for p in params) else None
            ops.sample(logits, out, fd[0], nucleus, idv[0], idv[1], logprob_out=lp)
        host_tokens, host_lp, event = self._host_buffers(n)
        host_tokens[:n].copy_(out, non_blocking=True)
        if lp is not None:
            host_lp[:n].copy_(lp, non_blocking=True)
        event.record()
        self.bytes_read += 4 * n * (2 if lp is not None else 1)
        return PendingSample(n, host_tokens, host_lp if lp is not None else None, event)
