"""Packing collator (reference: ironcore/dataloader/collator.py:17-255)."""

from ironcore_b200.data.collator import UniversalCollator, create_collator, first_fit_decreasing  # noqa: F401
