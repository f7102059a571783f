"""Parts a layer is put together from, and their registration."""
from ..registry import register_part
from .attention import GQAAttention
from .base import Block, BuildContext, CacheSpec, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .mlp import SwiGLUMLP
from .norm import RMSNorm
from .rope import RotaryEmbedding

register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rope", RotaryEmbedding)
register_part("mixer", "gqa_attention", GQAAttention)
register_part("feed_forward", "swiglu", SwiGLUMLP)
register_part("block", "prenorm", PreNormBlock)

__all__ = ["Block", "BuildContext", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "LMHead", "TokenEmbedding", "SwiGLUMLP", "RMSNorm", "RotaryEmbedding", "GQAAttention"]
