"""Dataset serialisation (reference: ironcore/preprocessing/__init__.py)."""

from ironcore_b200.data.serializer import DataSerializer  # noqa: F401

__all__ = ["DataSerializer"]
