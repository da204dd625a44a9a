"""Positional embeddings (reference: ironcore/layers/positional_embedding/__init__.py)."""

from ironcore_b200.layers.positional import SinusoidalPositionalEmbedding  # noqa: F401

from .absolute import PositionalEncoding
from .rotary import RotaryPositionalEmbedding

__all__ = ["PositionalEncoding", "RotaryPositionalEmbedding"]
