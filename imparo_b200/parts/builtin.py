"""Registers the built-in parts."""
from .attention import AttentionMixer
from .base import register_part
from .block import PreNormResidualBlock
from .embedding import LinearHead, TokenEmbedding
from .feedforward import SwiGLU
from .norm import RMSNorm
from .position import NoPosition, RotaryNeox
from .shortconv import ShortConvMixer

register_part("mixer", "attention", AttentionMixer, replace=True)
register_part("mixer", "short_conv", ShortConvMixer, replace=True)
register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("position", "rope_neox", RotaryNeox, replace=True)
register_part("position", "none", NoPosition, replace=True)
register_part("block", "prenorm_residual", PreNormResidualBlock, replace=True)
register_part("embedding", "token_table", TokenEmbedding, replace=True)
register_part("head", "linear", LinearHead, replace=True)
