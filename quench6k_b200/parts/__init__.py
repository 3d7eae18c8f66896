from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheRequest, FeedForward, LayerCache,
                   Mixer, Norm, Part, PositionEncoding, Runtime, make_part, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position_encoding, to_f32, to_operand)
from . import norm, position, attention, ffn, block   # noqa: F401  (register the built-in parts)
