"""Persistence: native checkpoints (resume, TP/EP merge and split) and HuggingFace interop."""

from .native import (HFConfigManager, find_latest_step, load_checkpoint, merge_model_parallel_state,
                     save_checkpoint)

__all__ = ["HFConfigManager", "find_latest_step", "load_checkpoint", "merge_model_parallel_state", "save_checkpoint"]


def __getattr__(name):
    if name in ("load_from_huggingface", "export_to_huggingface", "WeightMapper", "Architecture"):
        from . import hf_interop

        return getattr(hf_interop, name)
    raise AttributeError(name)
