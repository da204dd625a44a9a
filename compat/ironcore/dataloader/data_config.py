"""Dataset configuration (reference: ironcore/dataloader/data_config.py)."""

from ironcore_b200.data.data_config import DatasetConfig, UniversalDataConfig  # noqa: F401
