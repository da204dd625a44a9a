"""MLP (reference: ironcore/layers/mlp.py)."""

from ironcore_b200.layers.mlp import MLP  # noqa: F401
