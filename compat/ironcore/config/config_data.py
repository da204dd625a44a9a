"""Configuration group module of the reference (ironcore/config/config_data.py:18-59)."""

from ironcore_b200.config.schema import DataConfig  # noqa: F401
