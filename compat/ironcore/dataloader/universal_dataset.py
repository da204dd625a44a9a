"""Binary datasets and weighted mixing (reference: ironcore/dataloader/universal_dataset.py:20-200)."""

from ironcore_b200.data.dataset import BinaryDataset, WeightedMixingDataset  # noqa: F401
