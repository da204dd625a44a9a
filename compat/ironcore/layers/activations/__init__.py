"""Activations (reference: ironcore/layers/activations/activations.py:15-60)."""

from ironcore_b200.layers.activations import Activation, get_activation  # noqa: F401
