from .attention import PagedAttention
from .base import (CacheNeed, FeedForward, Mixer, Norm, PagedKVNeed, ParamSpec, Part, PositionEncoding,
                   StateNeed)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .ffn import SwiGLU
from .norm import RMSNorm
from .rope import RotaryEmbedding

__all__ = ["PagedAttention", "CacheNeed", "FeedForward", "Mixer", "Norm", "PagedKVNeed", "ParamSpec", "Part",
           "PositionEncoding", "StateNeed", "PreNormBlock", "OutputHead", "TokenEmbedding", "SwiGLU", "RMSNorm",
           "RotaryEmbedding"]
