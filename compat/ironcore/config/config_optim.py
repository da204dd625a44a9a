"""Configuration group module of the reference (ironcore/config/config_optim.py:17-61)."""

from ironcore_b200.config.schema import OptimConfig  # noqa: F401
