"""Configuration group module of the reference (ironcore/config/config.py:20-129)."""

from ironcore_b200.config.schema import BaseConfig, MainConfig  # noqa: F401
