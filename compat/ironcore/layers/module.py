"""Module base class (reference: ironcore/layers/module.py)."""

from ironcore_b200.layers.module import BaseModule  # noqa: F401
