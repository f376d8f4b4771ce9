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

    def forward(self, resid: torch.Tensor, pending: torch.Tensor | None, batch,
                cache: CacheView, write: bool) -> torch.Tensor:
        h = self.mixer_norm.forward(resid, pending)
        a = self.mixer.forward(h, batch, cache, write, self.position)
        h = self.feed_forward_norm.forward(resid, a)
        return self.feed_forward.forward(h)
