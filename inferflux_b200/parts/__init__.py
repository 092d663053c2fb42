"""The parts layers are made of.  Importing this package registers the
built-in kinds; more can be added with
:func:`inferflux_b200.config.registry.register_part`."""
from .base import Part, KVNeed, StateNeed, RunInfo
from .linear import Linear
from .norm import RMSNorm
from .position import RotaryHalf
from .attention import GQAttention
from .feed_forward import SwiGLU
from .block import PreNormBlock
from .embedding import TokenEmbedding, LinearHead

__all__ = ["Part", "KVNeed", "StateNeed", "RunInfo", "Linear", "RMSNorm", "RotaryHalf",
           "GQAttention", "SwiGLU", "PreNormBlock", "TokenEmbedding", "LinearHead"]
