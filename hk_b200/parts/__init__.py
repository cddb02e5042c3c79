from .attention import GQAAttention
from .base import (KVCacheSpec, MATRIX, ParamSpec, Part, Precision, StateSpec, StepTables, TABLE, VECTOR, part_class,
                   register_part)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .feed_forward import SwiGLUFeedForward
from .norm import RMSNorm
from .position import RopeScaling, RotaryEmbedding

__all__ = [
    "GQAAttention", "KVCacheSpec", "MATRIX", "OutputHead", "ParamSpec", "Part", "Precision", "PreNormBlock",
    "RMSNorm", "RopeScaling", "RotaryEmbedding", "StateSpec", "StepTables", "SwiGLUFeedForward", "TABLE", "TokenEmbedding", "VECTOR",
    "part_class", "register_part",
]
