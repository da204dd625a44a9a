"""Loss functions and the default forward step (reference: ironcore/training_utils.py:11-151)."""

from ironcore_b200.training_utils import (compute_token_accuracy, forward_step, get_batch, get_loss_func,  # noqa: F401
                                          loss_func, loss_func_sft)
