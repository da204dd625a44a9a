"""Positional embeddings (reference: ironcore/layers/positional_embedding/)."""

from ironcore_b200.layers.positional import RotaryPositionalEmbedding, SinusoidalPositionalEmbedding  # noqa: F401
