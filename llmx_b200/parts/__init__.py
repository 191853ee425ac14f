"""Parts a model is put together from."""
from .base import GroupView, Part, Precision, StepBatch
from .linear import Linear
from .norm import GroupedRMSNorm, LayerNorm, RMSNorm
from .rope import NoPositionEncoding, RotaryEmbedding
from .attention import Attention
from .mlp import ClampedGLU, GatedMLP, RoutedExperts, TableRoutedExperts
from .block import InputFilter, ParallelBlock, PreNormBlock, SandwichBlock
from .linear_attention import DecayedLinearAttention
from .delta_rule import GatedDeltaRule
from .latent_attention import LatentAttention
from .embedding import LogitsHead, PairHashEmbedding, TokenEmbedding
from .state_space import SelectiveStateSpace
from .masked_attention import MaskedAttention
from .mixer_pair import MixerPair

__all__ = ["GroupView", "Part", "Precision", "StepBatch", "Linear", "RMSNorm", "NoPositionEncoding",
           "RotaryEmbedding", "Attention", "GatedMLP", "PreNormBlock", "LogitsHead", "TokenEmbedding", "LayerNorm", "ClampedGLU",
           "ParallelBlock", "DecayedLinearAttention", "GatedDeltaRule", "LatentAttention",
           "TableRoutedExperts", "SelectiveStateSpace", "MaskedAttention", "MixerPair", "SandwichBlock",
           "GroupedRMSNorm", "RoutedExperts", "InputFilter", "PairHashEmbedding"]
