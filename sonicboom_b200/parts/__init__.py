"""Parts a layer is put together from: norms, position encodings, mixers, feed-forwards and
their arrangement in a block; each kind is looked up by name in a registry."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward,
                   Mixer, Norm, Part, PositionEncoding, StepContext, make, register_block,
                   register_feed_forward, register_mixer, register_norm,
                   register_position_encoding)
from . import norm, rotary, attention, feedforward, block  # noqa: F401  (fill the registries)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block",
           "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "StepContext", "make",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position_encoding"]
