"""Parts of a decoder (norm, position encoding, mixer, feed-forward, block, embedding, head)."""
from .base import (FixedStateSpec, MATRIX, NORM_WEIGHT, PagedKVSpec, Part, WeightSpec, build_part,
                   register_part)
from . import norm, rope, attention, mlp, block, embed_head  # noqa: F401  (register the parts)
from .attention import Attention
from .block import PreNormBlock
from .embed_head import Embedding, LMHead
from .mlp import SwiGLU
from .model import CausalLM
from .norm import RMSNorm
from .rope import NoPosition, RopeNeox, Rotation

__all__ = [
    "Attention", "CausalLM", "Embedding", "FixedStateSpec", "LMHead", "MATRIX", "NORM_WEIGHT", "NoPosition",
    "PagedKVSpec", "Part", "PreNormBlock", "RMSNorm", "RopeNeox", "Rotation", "SwiGLU", "WeightSpec",
    "build_part", "register_part",
]
