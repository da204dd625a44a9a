"""Layer building blocks (reference: ironcore/layers/*)."""

from ironcore_b200.layers.activations import Activation  # noqa: F401
from ironcore_b200.layers.attention import Attention  # noqa: F401
from ironcore_b200.layers.mlp import MLP  # noqa: F401
from ironcore_b200.layers.module import BaseModule  # noqa: F401
from ironcore_b200.layers.norm import FusedLayerNorm, FusedRMSNorm, get_norm  # noqa: F401
from ironcore_b200.layers.positional import RotaryPositionalEmbedding, SinusoidalPositionalEmbedding  # noqa: F401
