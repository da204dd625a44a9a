"""Dummy model (reference: ironcore/models/dummy.py)."""

from ironcore_b200.models.dummy import DummyModel  # noqa: F401
