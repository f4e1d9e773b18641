"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (KVNeed, StateNeed, LayerCache, StepContext, Part, Norm, PositionEncoding, Mixer, FeedForward, Block,
                   register_mixer, register_feed_forward, register_norm, register_position_encoding,
                   make_mixer, make_feed_forward, make_norm, make_position_encoding,
                   MIXERS, FEED_FORWARDS, NORMS, POSITION_ENCODINGS)
from .norm import RMSNorm
from .rotary import RotaryEncoding
from .attention import AttentionMixer
from .dense_ffn import SwiGLUFeedForward
from .moe_ffn import MoEFeedForward
from .block import PreNormBlock
