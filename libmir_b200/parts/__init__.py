"""Built-in parts and their registration by kind."""

from ..registry import register_part
from .attention import SoftmaxAttention
from .base import Block, BuildEnv, FeedForward, Mixer, Norm, Part, PartContext, Position, ScratchContext
from .block import ARRANGEMENTS, PreNormBlock, build_block
from .feed_forward import SwiGlu
from .norm import RmsNorm
from .rope import Rotary, inverse_frequencies

register_part("rms_norm", RmsNorm)
register_part("rotary", Rotary)
register_part("softmax_attention", SoftmaxAttention)
register_part("swiglu", SwiGlu)

__all__ = ["ARRANGEMENTS", "Block", "BuildEnv", "FeedForward", "Mixer", "Norm", "Part", "PartContext", "Position", "PreNormBlock", "RmsNorm",
           "Rotary", "ScratchContext", "SoftmaxAttention", "SwiGlu", "build_block", "inverse_frequencies"]
