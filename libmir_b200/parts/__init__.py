"""Built-in parts and their registration by kind."""

from ..registry import register_part
from .attention import SoftmaxAttention
from .base import Block, BuildEnv, FeedForward, Mixer, Norm, Part, PartContext, Position, ScratchContext
from .block import ARRANGEMENTS, ParallelBlock, PreNormBlock, build_block
from .delta_rule import GatedDeltaRule
from .feed_forward import GeluMlp, SwiGlu
from .side_by_side import SideBySide
from .norm import RmsNorm
from .rope import Rotary, inverse_frequencies

register_part("rms_norm", RmsNorm)
register_part("rotary", Rotary)
register_part("softmax_attention", SoftmaxAttention)
register_part("swiglu", SwiGlu)
register_part("gelu_mlp", GeluMlp)
register_part("gated_delta_rule", GatedDeltaRule)
register_part("side_by_side", SideBySide)

__all__ = ["ARRANGEMENTS", "Block", "BuildEnv", "FeedForward", "GatedDeltaRule", "GeluMlp", "Mixer", "Norm", "ParallelBlock", "Part",
           "PartContext", "Position", "PreNormBlock", "RmsNorm", "Rotary", "ScratchContext", "SideBySide", "SoftmaxAttention",
           "SwiGlu", "build_block", "inverse_frequencies"]
