"""Module base class (reference: ironcore/layers/module.py:19-232): ``BaseModule(config)`` with ``init_weights()``,
``device`` / ``dtype`` properties and profiler ranges around every submodule."""

from ironcore_b200.layers.module import BaseModule, init_parameters  # noqa: F401
