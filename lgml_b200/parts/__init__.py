from .attention import Attention
from .base import KINDS, Part, make_part, register_part, registered
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .mlp import GatedMLP
from .norm import RMSNorm
from .rope import NoPosition, Rope, RotaryPosition, frequency_factors, store_kv

__all__ = ["Attention", "KINDS", "Part", "make_part", "register_part", "registered", "PreNormBlock", "LMHead",
           "TokenEmbedding", "GatedMLP", "RMSNorm", "NoPosition", "Rope", "RotaryPosition", "frequency_factors", "store_kv"]
