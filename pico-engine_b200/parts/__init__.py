"""The parts layers are put together from, their registries, and the decoder built of them."""
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward, KVView, Mixer, Norm, Part,
                   Position, StepContext, build_part, register_arrangement, register_feed_forward, register_mixer,
                   register_norm, register_position)
from .norm import RMSNorm
from .position import NoPosition, RotaryHalf
from .attention import GQAAttention
from .feed_forward import SwiGLU
from .block import Layer, pre_norm
from .model import DecoderModel

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "FeedForward", "KVView", "Mixer", "Norm",
           "Part", "Position", "StepContext", "build_part", "register_arrangement", "register_feed_forward",
           "register_mixer", "register_norm", "register_position", "RMSNorm", "NoPosition", "RotaryHalf",
           "GQAAttention", "SwiGLU", "Layer", "pre_norm", "DecoderModel"]
