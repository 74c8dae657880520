"""The parts a model is put together from: norms, position encodings, mixers,
feed-forwards and their arrangement in a block."""

from .base import Part, build_part, register_part
from .norm import RMSNorm
from .rotary import NoPosition, RotaryHalf
from .attention import GQAAttention
from .mlp import GatedMLP
from .block import PreNormBlock

__all__ = ["Part", "build_part", "register_part", "RMSNorm", "RotaryHalf", "NoPosition",
           "GQAAttention", "GatedMLP", "PreNormBlock"]
