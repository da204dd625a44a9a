"""Configuration group module of the reference (ironcore/config/config_trainer.py:18-175)."""

from ironcore_b200.config.schema import InitConfig, OperationConfig, TrainerConfig  # noqa: F401
