"""Dataset serialisation to .bin / .idx (reference: ironcore/preprocessing/serializer.py:17-410)."""

from ironcore_b200.data.serializer import DataSerializer  # noqa: F401
