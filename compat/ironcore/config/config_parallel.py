"""Configuration group module of the reference (ironcore/config/config_parallel.py:18-48)."""

from ironcore_b200.config.schema import ParallelConfig  # noqa: F401
