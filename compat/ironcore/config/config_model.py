"""Configuration group module of the reference (ironcore/config/config_model.py:18-154)."""

from ironcore_b200.config.schema import ModelConfig, PositionalEmbeddingConfig  # noqa: F401
