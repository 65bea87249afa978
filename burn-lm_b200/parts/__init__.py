"""The parts layers are put together from: norm, position encoding, mixer, feed-forward, block,
embedding and head.  Importing this package registers the built-in kinds."""
from .base import CacheNeed, Part, Runtime, StepContext
from .linear import Linear
from .norm import RMSNorm, RMSNormSpec
from .position import Llama3Scaling, NoPosition, NoPositionSpec, Rotary, RotarySpec, rotary_inverse_frequencies
from .attention import Attention, AttentionSpec
from .feed_forward import SwiGLU, SwiGLUSpec
from .block import PreNormBlock
from .embedding import Embedding, EmbeddingSpec, Head, HeadSpec

__all__ = ["CacheNeed", "Part", "Runtime", "StepContext", "Linear", "RMSNorm", "RMSNormSpec", "Llama3Scaling",
           "NoPosition", "NoPositionSpec", "Rotary", "RotarySpec", "rotary_inverse_frequencies", "Attention",
           "AttentionSpec", "SwiGLU", "SwiGLUSpec", "PreNormBlock", "Embedding", "EmbeddingSpec", "Head", "HeadSpec"]
