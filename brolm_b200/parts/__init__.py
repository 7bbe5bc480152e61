from .attention import Attention
from .base import ParamSpec, Part, PartSpec, part_class, register_part, registered_parts
from .block import Block, BlockSpec, OneNormParallelBlock, ParallelBlock, PostNormBlock
from .experts import RoutedExperts
from .feedforward import DenseFeedForward, GatedFeedForward
from .latent_attention import LatentAttention
from .layout import EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, PairTableSpec
from .linear import linear
from .norm import Cast, RMSNorm, add_then_norm
from .position import RotaryEmbedding
from .recurrent import DecayLinearAttention, GatedRecurrence, SideBySide, StateSpace
from .stream import ConcatLinear

__all__ = ["Attention", "ParamSpec", "Part", "PartSpec", "part_class", "register_part", "registered_parts", "Block",
           "BlockSpec", "GatedFeedForward", "EmbeddingSpec", "HeadSpec", "LayerCall", "ModelLayout", "linear",
           "RMSNorm", "add_then_norm", "RotaryEmbedding", "ParallelBlock", "RoutedExperts", "LatentAttention",
           "PairTableSpec", "ConcatLinear", "PostNormBlock", "DenseFeedForward", "Cast", "GatedRecurrence", "SideBySide",
           "StateSpace", "DecayLinearAttention", "OneNormParallelBlock"]
