from .attention import Attention
from .base import (Block, BuildOptions, FeedForward, KVSpec, Mixer, Norm, Part, PositionEncoding, StateSpec)
from .block import HiddenStream, PreNormBlock
from .embedding import TokenEmbedding, VocabHead
from .feedforward import SwiGLU
from .linear import Linear
from .norm import RMSNorm
from .position import RotaryEncoding, scaled_inv_freq

__all__ = ["Attention", "Block", "BuildOptions", "FeedForward", "KVSpec", "Mixer", "Norm", "Part", "PositionEncoding",
           "StateSpec", "HiddenStream", "PreNormBlock", "TokenEmbedding", "VocabHead", "SwiGLU", "Linear",
           "RMSNorm", "RotaryEncoding", "scaled_inv_freq"]
