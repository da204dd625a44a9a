"""Optimizers and schedules: reference-rule AdamW, the flat-buffer distributed engine
(DP reduction, TP-aware clipping, ZeRO-1, host-offloaded moments) and distributed Muon."""

from .adam import AdamWOptimizer, adam_update_reference
from .distributed import DistributedOptimizer, is_muon_param, is_no_decay
from .lr_scheduler import (ConstantLRScheduler, CosineAnnealingLR, LinearDecayLRScheduler, get_lr_scheduler)
from .muon import MuonState, newton_schulz, newton_schulz_reference


def get_param_groups(config, model):
    """Two groups: decayed and not decayed (bias, norm gains, learned position tables)."""
    o = config.optim
    decay, no_decay = [], []
    seen = set()
    for _mn, mod in model.named_modules():
        for pn, p in mod.named_parameters(recurse=False):
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            (no_decay if is_no_decay(mod, pn, o.no_decay_on_embedding) else decay).append(p)
    return [{"params": decay, "weight_decay": o.weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


def get_optimizer(config, model, device_type=None, distributed: bool = True):
    """``distributed=True`` (default) returns the flat-buffer engine used by the trainer;
    ``False`` returns the plain per-parameter AdamW (``torch.optim.Optimizer`` API)."""
    name = config.optim.optimizer.lower()
    if name not in ("adam", "adamw", "muon"):
        raise NotImplementedError(f"optimizer {config.optim.optimizer} is not implemented")
    if distributed:
        return DistributedOptimizer(model, config)
    if name == "muon":
        raise NotImplementedError("Muon runs on the distributed engine (distributed=True)")
    o = config.optim
    return AdamWOptimizer(get_param_groups(config, model), lr=o.max_lr, betas=(o.adam_beta1, o.adam_beta2),
                          eps=o.adam_eps, weight_decay=o.weight_decay)


__all__ = ["AdamWOptimizer", "ConstantLRScheduler", "CosineAnnealingLR", "DistributedOptimizer",
           "LinearDecayLRScheduler", "MuonState", "adam_update_reference", "get_lr_scheduler", "get_optimizer",
           "get_param_groups", "is_muon_param", "is_no_decay", "newton_schulz", "newton_schulz_reference"]
