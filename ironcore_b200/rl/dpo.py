"""Direct preference optimisation on (chosen, rejected) pairs.

    L = -log sigmoid( beta * [ (log pi(y_c | x) - log pi_ref(y_c | x)) - (log pi(y_r | x) - log pi_ref(y_r | x)) ] )

with sequence log-probabilities summed over the response tokens (the positions the SFT mask keeps) and ``pi_ref``
a frozen copy of the policy taken when training starts. ``label_smoothing`` eps mixes in the loss of the flipped
pair (conservative DPO). The data side is the reference's: ``task_type: dpo`` datasets serialised as chosen /
rejected rows sharing a ``group_id`` and collated into ``chosen_*`` / ``rejected_*`` batches
(ironcore/preprocessing/serializer.py:293-326, ironcore/dataloader/collator.py:206-229); the reference stops
there (its ``forward_step`` reads ``input_ids`` / ``labels`` only), this module is the training step for it."""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from ..trainer import Trainer


def dpo_loss(policy_chosen: torch.Tensor, policy_rejected: torch.Tensor, ref_chosen: torch.Tensor,
             ref_rejected: torch.Tensor, beta: float = 0.1, label_smoothing: float = 0.0
             ) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Sequence log-probs [B] of the four (model, answer) combinations -> (mean loss, statistics)."""
    logits = beta * ((policy_chosen - ref_chosen) - (policy_rejected - ref_rejected))
    loss = -(1.0 - label_smoothing) * F.logsigmoid(logits) - label_smoothing * F.logsigmoid(-logits)
    with torch.no_grad():
        stats = {"reward_chosen": (beta * (policy_chosen - ref_chosen)).mean(),
                 "reward_rejected": (beta * (policy_rejected - ref_rejected)).mean(),
                 "reward_accuracy": (logits > 0).float().mean(), "margin": logits.mean() / max(beta, 1e-12)}
    return loss.mean(), stats


def sequence_logprobs(model, batch: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """Sum of the response-token log-probs of every row of the ``prefix`` (``chosen_`` / ``rejected_``) half of a
    DPO batch: [B]. Rows hold one sample each (the collator does not pack DPO pairs)."""
    ids, labels = batch[prefix + "input_ids"], batch[prefix + "labels"]
    mask = batch.get(prefix + "loss_mask")
    lp = model.token_logprobs(ids, labels)
    keep = (labels != -100).to(lp.device)
    if mask is not None:
        keep = keep & mask.to(lp.device).bool()
    return (lp * keep.to(lp.dtype)).sum(dim=-1)


class DPOTrainer(Trainer):
    """``Trainer`` whose step is the DPO loss on ``chosen_*`` / ``rejected_*`` batches. ``rl.dpo_beta`` and
    ``rl.dpo_label_smoothing`` configure the loss; everything else (parallel layouts, optimizer engine, schedules,
    checkpoints, logging) is the base trainer's."""

    def __init__(self, config, **kw):
        kw.setdefault("forward_step_func", self._forward_step)
        super().__init__(config, **kw)
        from .reference_policy import frozen_copy

        self.ref_model = frozen_copy(self.model, config, self.loss_fn, self.device)
        self.last_stats: Optional[Dict[str, float]] = None

    def _forward_step(self, model, data_iterator):
        batch = next(data_iterator)
        rl = self.config.rl
        with torch.no_grad():
            ref_c = sequence_logprobs(self.ref_model, batch, "chosen_")
            ref_r = sequence_logprobs(self.ref_model, batch, "rejected_")
        pol_c = sequence_logprobs(model, batch, "chosen_")
        pol_r = sequence_logprobs(model, batch, "rejected_")
        loss, stats = dpo_loss(pol_c, pol_r, ref_c, ref_r, rl.dpo_beta, rl.dpo_label_smoothing)
        self.last_stats = {k: float(v) for k, v in stats.items()}
        return loss

    def log_training(self, step, losses, grad_norm, param_norm):
        metrics = super().log_training(step, losses, grad_norm, param_norm)
        if self.last_stats:
            from .. import global_vars as G

            s = self.last_stats
            self.logger.info("          dpo | reward accuracy %.2f | chosen %.4f | rejected %.4f | margin %.3f",
                             s["reward_accuracy"], s["reward_chosen"], s["reward_rejected"], s["margin"])
            G.log_metrics({f"dpo/{k}": v for k, v in s.items()}, step + 1)
        return metrics

    @torch.no_grad()
    def _eval_loop(self, iterator, max_batches: int, tag: str, step: int):
        """Preference loss and reward accuracy over held-out pairs."""
        if iterator is None:
            return None
        from .. import global_vars as G

        rl = self.config.rl
        self.model.eval()
        losses, accs = [], []
        for i, batch in enumerate(iterator):
            if i >= max_batches:
                break
            lp = {(m, h): sequence_logprobs(model, batch, h) for m, model in (("p", self.model), ("r", self.ref_model))
                  for h in ("chosen_", "rejected_")}
            loss, stats = dpo_loss(lp["p", "chosen_"], lp["p", "rejected_"], lp["r", "chosen_"], lp["r", "rejected_"],
                                   rl.dpo_beta, rl.dpo_label_smoothing)
            losses.append(loss.float())
            accs.append(float(stats["reward_accuracy"]))
        self.model.train()
        if not losses:
            return None
        metrics = {f"{tag}_loss": self.average_loss(losses), f"{tag}_reward_accuracy": sum(accs) / len(accs)}
        self.logger.log_metrics(metrics, title=f"{tag} @ step {step + 1}")
        G.log_metrics(metrics, step + 1)
        return metrics
