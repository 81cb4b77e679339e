from .base import (
    Block,
    CacheSpec,
    FeedForward,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    StateSpec,
    WeightSpec,
    make_block,
    make_feed_forward,
    make_mixer,
    make_norm,
    make_position,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position,
)
from .params import (
    AttentionParams,
    Llama3Scaling,
    NoPositionParams,
    RMSNormParams,
    RopeParams,
    SwiGLUParams,
)
from . import attention, block, feed_forward, norm, position  # register the built-in parts

__all__ = [n for n in dir() if not n.startswith("_")]
