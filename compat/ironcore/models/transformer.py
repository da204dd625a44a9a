"""Transformer stack (reference: ironcore/models/transformer.py)."""

from ironcore_b200.models.transformer import TransformerLayer, TransformerModel  # noqa: F401
