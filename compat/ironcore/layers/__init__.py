"""Layer building blocks (reference: ironcore/layers/*), built from the configuration object."""

from ironcore_b200.layers.norm import FusedLayerNorm, FusedRMSNorm  # noqa: F401
from ironcore_b200.layers.positional import SinusoidalPositionalEmbedding  # noqa: F401

from .activations import Activation, GLUActivation, get_activation  # noqa: F401
from .attention import Attention  # noqa: F401
from .embedding import LanguageModelEmbedding  # noqa: F401
from .layernorm import LayerNorm, RmsNorm, get_norm  # noqa: F401
from .mlp import MLP  # noqa: F401
from .module import BaseModule  # noqa: F401
from .positional_embedding import PositionalEncoding, RotaryPositionalEmbedding  # noqa: F401
