"""Parts a layer is put together from: mixer, feed-forward, norm, position encoding, block."""

from . import attention, block, feed_forward, norm, position  # noqa: F401  (registration)
from .base import (Block, BuildContext, CacheView, FeedForward, KVSpec, Mixer, Norm, Part,
                   PositionEncoding, StateSpec)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position_encoding)

__all__ = ["BLOCKS", "Block", "BuildContext", "CacheView", "FEED_FORWARDS", "FeedForward", "KVSpec",
           "MIXERS", "Mixer", "NORMS", "Norm", "POSITION_ENCODINGS", "Part",
           "PositionEncoding", "StateSpec", "make", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding"]
