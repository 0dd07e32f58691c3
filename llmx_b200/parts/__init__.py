"""Parts a model is put together from."""
from .base import GroupView, Part, Precision, StepBatch
from .linear import Linear
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEmbedding
from .attention import Attention
from .mlp import GatedMLP
from .block import PreNormBlock
from .embedding import LogitsHead, TokenEmbedding

__all__ = ["GroupView", "Part", "Precision", "StepBatch", "Linear", "RMSNorm", "NoPositionEncoding",
           "RotaryEmbedding", "Attention", "GatedMLP", "PreNormBlock", "LogitsHead", "TokenEmbedding"]
