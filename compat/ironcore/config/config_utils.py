"""Configuration group module of the reference (ironcore/config/config_utils.py:18-65)."""

from ironcore_b200.config.schema import UtilsConfig  # noqa: F401
