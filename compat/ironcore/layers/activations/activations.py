"""Activations (reference: ironcore/layers/activations/activations.py:15-60). The gated forms follow the
published definitions (no learned linear map inside the activation)."""

from torch import nn

from ironcore_b200.layers.activations import Activation, canonical_activation, is_glu  # noqa: F401


class GLUActivation(Activation):
    """Gated activation on the two halves ``[feature | gate]`` of the last dimension."""

    def __init__(self, input_dim: int = 0, variant: str = "glu"):
        super().__init__(variant)
        self.input_dim, self.variant = input_dim, variant.lower()


def get_activation(activation_name: str, input_dim: int = None) -> nn.Module:
    if is_glu(activation_name):
        return GLUActivation(input_dim or 0, activation_name)
    return Activation(activation_name)
