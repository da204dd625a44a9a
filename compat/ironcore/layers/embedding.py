"""Embedding layer (reference: ironcore/layers/embedding.py)."""

from ironcore_b200.layers.embedding import LanguageModelEmbedding  # noqa: F401
