"""Arrangements of a layer's parts around the residual stream.

``pre_norm``: ``x + Mixer(Norm(x))`` then ``x + FeedForward(Norm(x))``
(src/scratch_llm/model.py:423-436 of the reference).  The residual stream is a 32-bit tensor
that every norm call updates in place: a block returns its last delta as *pending*, and the
next norm (the next block's, or the model's final norm) adds it while it reads the stream, so
the sum costs no pass of its own.
"""

from __future__ import annotations

import torch

from .base import Block, CacheView, FeedForward, Mixer, Norm, PositionEncoding
from .registry import register_block
from .stream import StreamSink


@register_block("pre_norm")
class PreNormBlock(Block):
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm",
             "feed_forward_norm": "norm", "position": "position"}
    pad_safe = True   # the arrangement itself touches no token: its parts decide

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm, position: PositionEncoding) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.position = position

    #: forward() takes next_entry=: what follows this block in the run order
    takes_next_entry = True

    def entry(self):
        """(the norm that takes the pending delta, the part that takes the norm's output)."""
        return self.mixer_norm, self.mixer

    @staticmethod
    def _sink(resid: torch.Tensor, producer, norm, consumer, n_tokens: int):
        """A sink for ``producer``'s output if it, the norm after it and the part after that
        all can hand the norm over (scratch_llm_b200.parts.stream), else None."""
        if n_tokens > StreamSink.MAX_TOKENS:    # (first: larger steps should pay nothing here)
            return None
        if norm is None or consumer is None or not getattr(producer, "accepts_sink", False) \
                or not getattr(norm, "deferrable", False):
            return None
        can = getattr(consumer, "accepts_normed", None)
        return StreamSink(resid, norm) if can is not None and can(n_tokens) else None

    def forward(self, resid: torch.Tensor, pending, batch, cache: CacheView, write: bool,
                next_entry=None):
        n = resid.shape[0]
        h = self.mixer_norm.forward(resid, pending)
        sink = self._sink(resid, self.mixer, self.feed_forward_norm, self.feed_forward, n)
        if sink is None:
            a = self.mixer.forward(h, batch, cache, write, self.position)
        else:
            a = self.mixer.forward(h, batch, cache, write, self.position, sink=sink)
        h = self.feed_forward_norm.forward(resid, a)
        norm, consumer = next_entry if next_entry is not None else (None, None)
        sink = self._sink(resid, self.feed_forward, norm, consumer, n)
        if sink is None:
            return self.feed_forward.forward(h)
        return self.feed_forward.forward(h, sink=sink)
