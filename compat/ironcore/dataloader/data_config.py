"""Dataset configuration (reference: ironcore/dataloader/data_config.py:15-231)."""

from ironcore_b200.data.data_config import (DataConfig, DatasetConfig, UniversalDataConfig,  # noqa: F401
                                            load_data_config)
