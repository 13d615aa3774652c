"""Parts a model is assembled from: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (CacheView, FeedForward, Mixer, Norm, NormedStream, PagedBuffer, PagedSpec, StreamState, Part, PositionEncoding, StateSpec,
                   TensorSpec, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make_part,
                   register_feed_forward, register_mixer, register_norm, register_position_encoding)
from .norm import RMSNorm
from .rope import RotaryEncoding
from .attention import GQAttention
from .shortconv import ShortConv
from .feedforward import SwiGLU
from .embedding import OutputHead, TokenEmbedding
from .block import BLOCKS, PreNormBlock, register_block

__all__ = [
    "CacheView", "FeedForward", "Mixer", "Norm", "NormedStream", "PagedBuffer", "PagedSpec", "StreamState", "Part", "PositionEncoding", "StateSpec",
    "TensorSpec", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "BLOCKS", "make_part",
    "register_feed_forward", "register_mixer", "register_norm", "register_position_encoding",
    "register_block", "RMSNorm", "RotaryEncoding", "GQAttention", "ShortConv", "SwiGLU", "OutputHead",
    "TokenEmbedding", "PreNormBlock",
]
