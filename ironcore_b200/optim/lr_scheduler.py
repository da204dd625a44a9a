"""Learning-rate schedules. The step counter is ``t = completed optimizer steps + 1``:
construction performs one ``step()`` so the first update already uses ``lr(t=1)``.
cosine: linear warm-up ``t / warmup`` while ``t <= warmup``, cosine from max to min over
``annealing_steps``, then ``min_lr``.
(Behavioural reference: ironcore/optimizer/lr_scheduler.py:19-133; the linear schedule is
implemented here as a working class.)"""

from __future__ import annotations

import math


class _Schedule:
    def __init__(self, optimizer, max_lr: float, min_lr: float, warmup_steps: int, annealing_steps: int,
                 total_steps: int):
        if max_lr < min_lr:
            raise ValueError("max_lr should be larger than min_lr")
        self.optimizer = optimizer
        self.max_lr, self.min_lr = max_lr, min_lr
        self.warmup_steps, self.annealing_steps, self.total_steps = warmup_steps, annealing_steps, total_steps
        self.base_lrs = [g.get("initial_lr", g.get("base_lr", max_lr)) for g in optimizer.param_groups]
        for g, b in zip(optimizer.param_groups, self.base_lrs):
            g.setdefault("initial_lr", b)
        self.last_epoch = -1
        self._step_count = 0
        self.step()

    def factor(self, t: int) -> float:  # fraction of (base - min) above min
        raise NotImplementedError

    def lr_at(self, t: int, base: float) -> float:
        if self.warmup_steps > 0 and t <= self.warmup_steps:
            return base * t / self.warmup_steps
        if t >= self.annealing_steps + self.warmup_steps:
            return self.min_lr
        return self.min_lr + (base - self.min_lr) * self.factor(t)

    def get_lr(self):
        return [self.lr_at(self._step_count, b) for b in self.base_lrs]

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def step(self, epoch=None):
        self.last_epoch = self.last_epoch + 1 if epoch is None else epoch
        self._step_count = self.last_epoch + 1
        for g, lr in zip(self.optimizer.param_groups, self.get_lr()):
            g["lr"] = lr * g.get("lr_mult", 1.0)

    def state_dict(self):
        return {"last_epoch": self.last_epoch, "_step_count": self._step_count, "base_lrs": list(self.base_lrs)}

    def load_state_dict(self, sd):
        self.last_epoch = sd["last_epoch"]
        self._step_count = sd.get("_step_count", self.last_epoch + 1)
        for g, lr in zip(self.optimizer.param_groups, self.get_lr()):
            g["lr"] = lr * g.get("lr_mult", 1.0)


class CosineAnnealingLR(_Schedule):
    def factor(self, t):
        return (1 + math.cos(math.pi * (t - self.warmup_steps) / self.annealing_steps)) / 2


class LinearDecayLRScheduler(_Schedule):
    def factor(self, t):
        return 1.0 - (t - self.warmup_steps) / self.annealing_steps


class ConstantLRScheduler(_Schedule):
    def lr_at(self, t, base):
        if self.warmup_steps > 0 and t <= self.warmup_steps:
            return base * t / self.warmup_steps
        return base


def get_lr_scheduler(config, optimizer):
    o = config.optim
    if o.annealing_steps == 0:
        o.annealing_steps = config.operation.train_steps
    kw = dict(max_lr=o.max_lr, min_lr=o.min_lr, warmup_steps=o.warmup_steps, annealing_steps=o.annealing_steps,
              total_steps=config.operation.train_steps)
    kind = o.lr_scheduler.lower()
    if kind == "cosine":
        return CosineAnnealingLR(optimizer, **kw)
    if kind == "linear":
        return LinearDecayLRScheduler(optimizer, **kw)
    if kind == "constant":
        return ConstantLRScheduler(optimizer, **kw)
    raise NotImplementedError(f"lr_scheduler {o.lr_scheduler} is not implemented")
