from .base import Param, Piece, Part, PagedKV, PagedTensors, FixedState, CacheView, StepShape, MixerPlan
from .registry import register, make, MIXERS, FEED_FORWARDS, NORMS, POSITIONS
from .norm import RMSNorm
from .rotary import Rotary, NoPosition
from .attention import GQAAttention
from .mlp import GatedMLP
from .embedding import TokenEmbedding, OutputHead
from .block import PreNormBlock

__all__ = ["Param", "Piece", "Part", "PagedKV", "PagedTensors", "FixedState", "CacheView", "StepShape", "MixerPlan", "register", "make", "MIXERS",
           "FEED_FORWARDS", "NORMS", "POSITIONS", "RMSNorm", "Rotary", "NoPosition", "GQAAttention",
           "GatedMLP", "TokenEmbedding", "OutputHead", "PreNormBlock"]
