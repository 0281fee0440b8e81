from .base import (Arena, Block, FeedForward, GroupStepView, Mixer, Norm, Part, PartSpec,
                   PositionEncoding, StepContext, register, NORMS, POSITION_ENCODINGS, MIXERS,
                   FEED_FORWARDS, BLOCKS)
from .norm import RMSNorm
from .rope import NeoxRope
from .attention import GQAAttention
from .mlp import SwiGLU
from .block import PreNormBlock

__all__ = ["Arena", "Block", "FeedForward", "GroupStepView", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "StepContext", "register", "NORMS", "POSITION_ENCODINGS", "MIXERS",
           "FEED_FORWARDS", "BLOCKS", "RMSNorm", "NeoxRope", "GQAAttention", "SwiGLU",
           "PreNormBlock"]
