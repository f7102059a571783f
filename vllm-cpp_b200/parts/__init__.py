"""Parts a layer is put together from, and their registration."""
from ..registry import register_part
from .attention import GQAAttention
from .base import Block, BuildContext, CacheSpec, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock
from .embedding import Embedding, Head, LMHead, TokenEmbedding
from .mlp import SwiGLUMLP
from .norm import RMSNorm
from .rope import RotaryEmbedding

register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rope", RotaryEmbedding)
register_part("mixer", "gqa_attention", GQAAttention)
register_part("feed_forward", "swiglu", SwiGLUMLP)
register_part("block", "prenorm", PreNormBlock)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)

__all__ = ["Block", "BuildContext", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "Embedding", "Head", "LMHead", "TokenEmbedding", "SwiGLUMLP", "RMSNorm", "RotaryEmbedding", "GQAAttention"]
