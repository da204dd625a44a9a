"""Native checkpoints (reference: ironcore/checkpointing/native.py)."""

from ironcore_b200.checkpoint.native import (HFConfigManager, find_latest_step, load_checkpoint,  # noqa: F401
                                              merge_model_parallel_state, save_checkpoint)
