"""Absolute positional embeddings (reference: ironcore/layers/positional_embedding/absolute.py)."""

from ironcore_b200.layers.positional import SinusoidalPositionalEmbedding  # noqa: F401
