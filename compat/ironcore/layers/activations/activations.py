"""Activations (reference: ironcore/layers/activations/activations.py:15-60)."""

from ironcore_b200.layers.activations import Activation, canonical_activation, get_activation, is_glu  # noqa: F401
