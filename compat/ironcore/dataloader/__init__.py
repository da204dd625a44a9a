"""Data iterators (reference: ironcore/dataloader/__init__.py:14-72)."""

from ironcore_b200.data import get_data_iterator  # noqa: F401
from ironcore_b200.data.collator import UniversalCollator  # noqa: F401
from ironcore_b200.data.data_config import DatasetConfig, UniversalDataConfig  # noqa: F401
from ironcore_b200.data.dataset import BinaryDataset, WeightedMixingDataset  # noqa: F401
