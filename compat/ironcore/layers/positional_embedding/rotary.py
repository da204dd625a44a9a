"""Rotary positional embedding (reference: ironcore/layers/positional_embedding/rotary.py)."""

from ironcore_b200.layers.positional import RotaryPositionalEmbedding  # noqa: F401
