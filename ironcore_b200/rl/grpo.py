"""GRPO pieces: synthetic deterministic reward, group-normalised advantages, the loss.

Loss over generated tokens: ``-min(rho * A, clip(rho, 1 - eps, 1 + eps) * A) + beta * KL`` with
``rho = exp(log pi_theta - log pi_old)`` (``pi_old`` = the detached rollout log-probs: one policy
update per rollout batch) and the k3 estimator ``KL = exp(delta) - delta - 1``,
``delta = log pi_ref - log pi_theta`` against a frozen copy of the initial policy. Advantages are
``(r - mean_group) / (std_group + eps)`` broadcast over a sequence's generated tokens.
(No counterpart in the reference.)"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops as RO


class VocabSubsetReward:
    """Reward = fraction of generated ids that fall in a fixed, seeded subset of the vocabulary."""

    def __init__(self, vocab_size: int, subset_size: int = 1024, seed: int = 7, device="cpu"):
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        ids = torch.randperm(vocab_size, generator=g)[:subset_size]
        table = torch.zeros(vocab_size, dtype=torch.bool)
        table[ids] = True
        self.table = table.to(device)

    def __call__(self, generated: torch.Tensor) -> torch.Tensor:
        """generated [S, N] token ids -> rewards [S] fp32."""
        return self.table.to(generated.device)[generated].float().mean(dim=-1)


def group_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-6) -> torch.Tensor:
    """rewards [num_prompts * group_size] (samples of one prompt contiguous) -> advantages, same shape."""
    r = rewards.view(-1, group_size)
    mean = r.mean(dim=1, keepdim=True)
    std = r.std(dim=1, keepdim=True, unbiased=False)
    return ((r - mean) / (std + eps)).reshape(-1)


def grpo_loss(logp: torch.Tensor, logp_old: torch.Tensor, logp_ref: Optional[torch.Tensor], advantages: torch.Tensor,
              mask: torch.Tensor, clip_eps: float = 0.2, kl_beta: float = 0.04) -> Tuple[torch.Tensor, dict]:
    """logp, logp_old, logp_ref, mask: [S, N]; advantages [S]. Returns (scalar loss, stats)."""
    s, n = logp.shape
    adv = advantages[:, None].expand(s, n).reshape(-1).float()
    tok_loss, ratio, kl = RO.grpo_token_loss(logp.reshape(-1).float(), logp_old.reshape(-1).float(),
                                             None if logp_ref is None else logp_ref.reshape(-1).float(), adv,
                                             mask.reshape(-1).float(), clip_eps, kl_beta)
    denom = mask.float().sum().clamp_min(1.0)
    loss = tok_loss.sum() / denom
    m = mask.reshape(-1).float()
    stats = {"ratio_mean": float((ratio * m).sum() / denom), "kl_mean": float((kl * m).sum() / denom)}
    return loss, stats
