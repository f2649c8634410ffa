"""Parts a layer is put together from, and their registration."""
from ..registry import register_part
from .attention import GQAAttention
from .base import Block, BuildContext, CacheSpec, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock
from .embedding import Embedding, Head, LMHead, SinusoidalTokenEmbedding, TokenEmbedding
from .gated_block import GatedPostNormBlock
from .mlp import DenseMLP, SwiGLUMLP
from .window_attention import ConvWindowAttention
from .norm import RMSNorm
from .rope import RotaryEmbedding

register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rope", RotaryEmbedding)
register_part("mixer", "gqa_attention", GQAAttention)
register_part("feed_forward", "swiglu", SwiGLUMLP)
register_part("block", "prenorm", PreNormBlock)
register_part("mixer", "conv_window_attention", ConvWindowAttention)
register_part("feed_forward", "dense", DenseMLP)
register_part("block", "gated_postnorm", GatedPostNormBlock)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "sinusoidal_token_embedding", SinusoidalTokenEmbedding)
register_part("head", "lm_head", LMHead)

__all__ = ["Block", "BuildContext", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "Embedding", "Head", "LMHead", "TokenEmbedding", "SwiGLUMLP", "DenseMLP", "GatedPostNormBlock",
           "ConvWindowAttention", "SinusoidalTokenEmbedding", "RMSNorm", "RotaryEmbedding", "GQAAttention"]
