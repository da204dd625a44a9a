"""Per-parameter AdamW with the reference's exact update rule: fp32 moments regardless of
the parameter dtype, ``denom = sqrt(v) + eps``, ``step_size = lr * sqrt(1 - b2^t) / (1 - b1^t)``,
decoupled decay ``p *= 1 - lr * wd``, update applied directly to the (16-bit) parameter —
no fp32 master copy. On CUDA each parameter is one fused kernel launch.
(Behavioural reference: ironcore/optimizer/optimizer.py:16-114.)"""

from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ..ops import kernels


def adam_update_reference(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """In-place reference update on any device (fp32 math)."""
    gf = g.float() * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    step_size = lr * math.sqrt(1.0 - beta2 ** step) / (1.0 - beta1 ** step)
    pf = p.float()
    if weight_decay != 0:
        pf.mul_(1 - lr * weight_decay)
    pf.addcdiv_(m, v.sqrt().add_(eps), value=-step_size)
    p.copy_(pf.to(p.dtype))


class AdamWOptimizer(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, **_unused):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.state_dtype = torch.float32

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=self.state_dtype)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=self.state_dtype)
                st["step"] += 1
                kw = dict(lr=group["lr"], beta1=b1, beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"],
                          step=st["step"], grad_scale=grad_scale)
                if p.is_cuda and p.is_contiguous() and g.is_contiguous():
                    kernels.adam_step_(p, g, st["exp_avg"], st["exp_avg_sq"], **kw)
                else:
                    adam_update_reference(p, g, st["exp_avg"], st["exp_avg_sq"], **kw)
        return loss

    def zero_grad(self, set_to_none: bool = False):
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    if set_to_none:
                        p.grad = None
                    else:
                        p.grad.detach_()
                        p.grad.zero_()
        return self
