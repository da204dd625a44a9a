"""Optimizers and schedules (reference: ironcore/optimizer/{__init__,optimizer,lr_scheduler}.py)."""

from ironcore_b200.optim import get_lr_scheduler, get_optimizer  # noqa: F401
from ironcore_b200.optim.adam import AdamWOptimizer  # noqa: F401

from .lr_scheduler import CosineAnnealingLR, LinearDecayLRScheduler  # noqa: F401
