"""Attention layer (reference: ironcore/layers/attention.py)."""

from ironcore_b200.layers.attention import Attention  # noqa: F401
