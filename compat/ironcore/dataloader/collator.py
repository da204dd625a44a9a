"""Packing collator (reference: ironcore/dataloader/collator.py)."""

from ironcore_b200.data.collator import UniversalCollator  # noqa: F401
