"""Parts that layers are put together from; importing this package registers the built-in kinds."""
from .base import (Block, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, Rotary, Runtime, StateNeed, kinds, make,
                   register_block, register_feed_forward, register_mixer, register_norm, register_position)
from .attention import GQAAttention
from .block import PreNormBlock
from .embedding import Embedding, Head
from .feed_forward import GatedFeedForward, MLP, SwiGLU
from .linear import Linear
from .norm import RMSNorm
from .position import NoPosition, Rope
