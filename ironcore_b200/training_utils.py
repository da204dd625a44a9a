"""Loss reductions, batch plumbing and token accuracy.
(Behavioural reference: ironcore/training_utils.py:11-151.)"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .models.language_model import IGNORE_INDEX, masked_mean_loss
from .parallel import mesh


def loss_func(per_token_loss: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
    """Pre-training reduction: sum(loss * mask) / sum(mask) over the micro-batch."""
    return masked_mean_loss(per_token_loss, loss_mask)


def loss_func_sft(per_token_loss: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
    """SFT reduction: mean over each sample's unmasked tokens, then mean over samples."""
    mask = loss_mask.float()
    per_sample = (per_token_loss.float() * mask).sum(-1) / mask.sum(-1).clamp_min(1.0)
    valid = (mask.sum(-1) > 0).float()
    return (per_sample * valid).sum() / valid.sum().clamp_min(1.0)


def get_loss_func(task_type: str):
    return loss_func_sft if str(task_type).lower() in ("sft", "dpo") else loss_func


def get_batch(data_iterator):
    batch = next(data_iterator)
    return batch


def forward_step(model, data_iterator):
    """One micro-batch forward; passes through the optional SFT fields the collator emits."""
    batch = get_batch(data_iterator)
    kwargs = {}
    for key in ("position_ids", "cu_seqlens", "loss_mask"):
        if key in batch and batch[key] is not None:
            kwargs[key] = batch[key]
    if batch.get("attention_mask") is not None and "cu_seqlens" not in kwargs:
        m = batch["attention_mask"]           # [rows, S, S] block mask of the packed samples
        kwargs["attn_mask"] = m.unsqueeze(1) if m.dim() == 3 else m
    return model(batch["input_ids"], batch["labels"], **kwargs)


@torch.no_grad()
def compute_token_accuracy(logits: torch.Tensor, labels: torch.Tensor, loss_mask=None, tp_group="default") -> float:
    """Fraction of counted positions whose arg-max (over the full, possibly sharded, vocab) equals the
    label. Counted: labels other than -100, and where ``loss_mask`` (optional, [B, S]) is non-zero."""
    if isinstance(loss_mask, str) or (loss_mask is not None and not torch.is_tensor(loss_mask)):
        loss_mask, tp_group = None, loss_mask      # (logits, labels, tp_group) positional form
    group = mesh.get_tensor_model_parallel_group() if tp_group == "default" else tp_group
    v_local = logits.shape[-1]
    vals, idx = logits.float().max(dim=-1)
    tp = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    if tp > 1:
        idx = idx + dist.get_rank(group) * v_local
        all_vals = [torch.empty_like(vals) for _ in range(tp)]
        all_idx = [torch.empty_like(idx) for _ in range(tp)]
        dist.all_gather(all_vals, vals.contiguous(), group=group)
        dist.all_gather(all_idx, idx.contiguous(), group=group)
        best = torch.stack(all_vals).argmax(dim=0, keepdim=True)
        idx = torch.stack(all_idx).gather(0, best).squeeze(0)
    mask = labels != IGNORE_INDEX
    if loss_mask is not None:
        mask = mask & (loss_mask > 0)
    correct = ((idx == labels) & mask).sum().item()
    return correct / max(int(mask.sum().item()), 1)
