"""Activation registry (reference: ironcore/layers/activations/__init__.py)."""

from .activations import Activation, GLUActivation, get_activation  # noqa: F401
