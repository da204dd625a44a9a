"""Learning-rate schedules with the reference's constructor argument order
(reference: ironcore/optimizer/lr_scheduler.py:19-133)."""

from ironcore_b200.optim import lr_scheduler as _s
from ironcore_b200.optim.lr_scheduler import ConstantLRScheduler, get_lr_scheduler  # noqa: F401


class CosineAnnealingLR(_s.CosineAnnealingLR):
    """``CosineAnnealingLR(optimizer, warmup_steps, annealing_steps, total_steps, max_lr, min_lr)``: linear warm-up,
    cosine from each group's base rate to ``min_lr`` over ``annealing_steps``, then ``min_lr``. Construction
    performs the first ``step()``. ``last_epoch`` other than -1 resumes at that step count."""

    def __init__(self, optimizer, warmup_steps: int, annealing_steps: int, total_steps: int, max_lr: float = 1e-5,
                 min_lr: float = 1e-8, last_epoch: int = -1):
        super().__init__(optimizer, max_lr=max_lr, min_lr=min_lr, warmup_steps=warmup_steps,
                         annealing_steps=annealing_steps, total_steps=total_steps)
        if last_epoch != -1:
            self.step(last_epoch)


class LinearDecayLRScheduler(_s.LinearDecayLRScheduler):
    """``LinearDecayLRScheduler(optimizer, warmup_steps, total_steps)``: linear warm-up, then linear decay to zero
    at ``total_steps``."""

    def __init__(self, optimizer, warmup_steps: int, total_steps: int):
        base = max(g.get("initial_lr", g["lr"]) for g in optimizer.param_groups)
        super().__init__(optimizer, max_lr=base, min_lr=0.0, warmup_steps=warmup_steps,
                         annealing_steps=max(total_steps - warmup_steps, 1), total_steps=total_steps)
