"""Data iterators (reference: ironcore/dataloader/__init__.py:14-72)."""

from ironcore_b200.data import get_data_iterator  # noqa: F401

from .collator import UniversalCollator, create_collator  # noqa: F401
from .data_config import DataConfig, DatasetConfig, UniversalDataConfig, load_data_config  # noqa: F401
from .universal_dataset import BinaryDataset, WeightedMixingDataset  # noqa: F401
