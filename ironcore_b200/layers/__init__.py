from .activations import Activation, get_activation, is_glu
from .attention import Attention
from .embedding import LanguageModelEmbedding
from .mlp import MLP
from .module import BaseModule
from .norm import FusedLayerNorm, FusedRMSNorm, Norm, get_norm
from .positional import RotaryPositionalEmbedding, SinusoidalPositionalEmbedding

__all__ = ["Activation", "Attention", "BaseModule", "FusedLayerNorm", "FusedRMSNorm", "LanguageModelEmbedding", "MLP",
           "Norm", "RotaryPositionalEmbedding", "SinusoidalPositionalEmbedding", "get_activation", "get_norm", "is_glu"]
