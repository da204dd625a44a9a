"""Cadence predicates of the training loop (reference: ironcore/controller.py:12-78)."""

from ironcore_b200.controller import TrainingControl  # noqa: F401
