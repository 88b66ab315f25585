"""Parts that layers are put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (Block, CacheSpec, FeedForward, LayerSlot, Mixer, Norm, Part, PositionEncoding, StateSpec,
                   StepContext, make_part, part_kinds, register_part)
from .linear import GroupedLinear, Linear
from .norm import L2Norm, RMSNorm
from .position import NoPositionEncoding, RotaryEncoding, rotary_inv_freq
from .attention import PagedAttention
from .feedforward import DenseSwiGLU, MoESigmoidTop1
from .block import PreNormBlock

__all__ = ["Block", "CacheSpec", "FeedForward", "LayerSlot", "Mixer", "Norm", "Part", "PositionEncoding",
           "StateSpec", "StepContext", "make_part", "part_kinds", "register_part", "GroupedLinear", "Linear",
           "L2Norm", "RMSNorm", "NoPositionEncoding", "RotaryEncoding", "rotary_inv_freq", "PagedAttention",
           "DenseSwiGLU", "MoESigmoidTop1", "PreNormBlock"]
