"""``Trainer(config, forward_step_func, loss_fn)`` (reference: ironcore/trainer.py:55-549)."""

from ironcore_b200.trainer import Trainer  # noqa: F401
