"""Learning-rate schedules (reference: ironcore/optimizer/lr_scheduler.py)."""

from ironcore_b200.optim.lr_scheduler import (ConstantLRScheduler, CosineAnnealingLR, LinearDecayLRScheduler,  # noqa: F401
                                              get_lr_scheduler)
