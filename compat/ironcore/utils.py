"""Helpers the reference keeps in ``ironcore/utils.py`` (:24-320): YAML loading, rank predicates, timers,
memory report, profiler ranges. ``clip_grad_norm_tp`` is not re-exported: gradient clipping is part of
the flat-buffer optimizers (``optimizer.step()`` returns the global norm it clipped to)."""

from ironcore_b200.config.loader import get_dataset_base_dir, load_yaml_config  # noqa: F401
from ironcore_b200.models.language_model import get_model_dtype  # noqa: F401
from ironcore_b200.parallel import mesh as _mesh
from ironcore_b200.utils.timers import Timer, get_memory_usage, profile_context, profile_function  # noqa: F401


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
    import torch

    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
