"""Helpers the reference keeps in ``ironcore/utils.py`` (:24-320): YAML loading, rank predicates, timers, memory
report, profiler ranges and the tensor-parallel-aware gradient clipping for plain ``.grad`` tensors (the
flat-buffer optimizers of ``ironcore_b200`` clip inside ``optimizer.step()`` and do not need it)."""

import os
import re
from typing import Iterable, Union

import torch
import torch.distributed as dist

from ironcore_b200.config import loader as _loader
from ironcore_b200.config.loader import get_dataset_base_dir  # noqa: F401
from ironcore_b200.models.language_model import get_model_dtype  # noqa: F401
from ironcore_b200.parallel import mesh as _mesh
from ironcore_b200.utils import timers as _timers
from ironcore_b200.utils.timers import Timer  # noqa: F401


def load_yaml_config(config_path):
    """YAML file -> dict with ``${VAR}`` interpolation and lists of single-key dicts merged into one dict."""
    return _loader.load_yaml_config(config_path)


def env_var_constructor(loader, node):
    """PyYAML constructor that substitutes ``${VAR}`` with the environment's value (empty when unset)."""
    value = loader.construct_scalar(node)
    return re.sub(r"\$\{(\w+)\}", lambda m: os.getenv(m.group(1), ""), value)


def is_first_rank() -> bool:
    return _mesh.get_rank() == 0


def is_last_rank() -> bool:
    return _mesh.get_rank() == _mesh.get_world_size() - 1


def print_rank_0(message: str) -> None:
    if is_first_rank():
        print(message, flush=True)


def print_last_rank(message: str) -> None:
    if is_last_rank():
        print(message, flush=True)


def get_device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def bytes_to_mib(bytes_value: int) -> int:
    return bytes_value // 1024 // 1024


def get_memory_usage(in_mib: bool = False) -> dict:
    """``memory_allocated / max_memory_allocated / memory_reserved / max_memory_reserved`` of the current CUDA
    device in bytes (MiB with ``in_mib``); empty without a GPU."""
    if not torch.cuda.is_available():
        return {}
    dev = torch.cuda.current_device()
    out = {"memory_allocated": torch.cuda.memory_allocated(dev), "max_memory_allocated": torch.cuda.max_memory_allocated(dev),
           "memory_reserved": torch.cuda.memory_reserved(dev), "max_memory_reserved": torch.cuda.max_memory_reserved(dev)}
    return {k: bytes_to_mib(v) for k, v in out.items()} if in_mib else out


def profile_function(tag):
    return _timers.profile_function(tag)


def profile_context(tag):
    return _timers.profile_context(tag)


def clip_grad_norm_tp(parameters: Union[torch.Tensor, Iterable[torch.Tensor]], max_norm: float,
                      norm_type: float = 2.0) -> torch.Tensor:
    """Clip the ``.grad`` tensors of ``parameters`` to a global norm of ``max_norm`` over the whole model: sharded
    parameters contribute their shard on every tensor-parallel rank, replicated ones are counted once. Returns the
    norm before clipping. ``norm_type``: 2 or ``inf``."""
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return torch.tensor(0.0)
    tp = _mesh.get_tensor_model_parallel_world_size()
    group = _mesh.get_tensor_model_parallel_group() if tp > 1 else None
    if float(norm_type) == float("inf"):
        total = torch.stack([p.grad.detach().abs().max() for p in params]).max()
        if group is not None:
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=group)
    elif float(norm_type) == 2.0:
        sq = params[0].grad.new_zeros((), dtype=torch.float32)
        for p in params:
            w = 1.0 if (tp == 1 or getattr(p, "tp_shard_dim", None) is not None) else 1.0 / tp
            sq = sq + w * p.grad.detach().float().pow(2).sum()
        if group is not None:
            dist.all_reduce(sq, group=group)
        total = sq.sqrt()
    else:
        raise ValueError("clip_grad_norm_tp supports the 2-norm and the infinity norm")
    coef = float(max_norm) / (total + 1e-6)
    if coef < 1:
        for p in params:
            p.grad.detach().mul_(coef.to(p.grad.dtype))
    return total
