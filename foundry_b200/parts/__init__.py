"""Layer parts and their registries; importing registers the built-in ones."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Part, Registry,
                   register_block, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding)
from . import attention, block, linear, mlp, norm, rope  # noqa: F401  (registration)
from .attention import GQAAttention
from .block import PreNormResidualBlock
from .linear import Linear, matmul_nt
from .mlp import SwiGLU
from .norm import RMSNorm
from .rope import Rope, RopeLlama3, llama3_inv_freq, plain_inv_freq

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Part", "Registry",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position_encoding", "GQAAttention", "PreNormResidualBlock", "Linear",
           "matmul_nt", "SwiGLU", "RMSNorm", "Rope", "RopeLlama3", "llama3_inv_freq",
           "plain_inv_freq"]
