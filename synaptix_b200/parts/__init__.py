from .attention import Attention
from .base import (FeedForward, Mixer, Norm, Part, PendingLinear, PendingNorm, PositionEncoding, Runtime, ScaledRows,
                   StepContext)
from .block import PreNormBlock
from .embedding import Embedding, OutputHead
from .linear import Linear
from .mlp import SwiGLU
from .norm import RMSNorm
from .rope import NoPosition, RotaryHalf, rotary_inv_freq

__all__ = ["Attention", "FeedForward", "Mixer", "Norm", "Part", "PendingLinear", "PendingNorm", "ScaledRows", "PositionEncoding", "Runtime",
           "StepContext", "PreNormBlock", "Embedding", "OutputHead", "Linear", "SwiGLU", "RMSNorm",
           "NoPosition", "RotaryHalf", "rotary_inv_freq"]
