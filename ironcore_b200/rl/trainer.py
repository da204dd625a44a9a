"""GRPO training loop: rollout on the paged-KV engine -> rewards -> group advantages -> one
clipped policy-gradient update (with a KL term to a frozen reference policy) per rollout batch.

Parallel layout: TP inside a replica (rollout and update share the sharded weights), DP across
replicas (each replica rolls out its share of the prompts; gradients are averaged by the
optimizer engine). Reported throughput = generated tokens per second of rollout time."""

from __future__ import annotations

import time
from typing import Dict

import torch
import torch.distributed as dist

from ..parallel import mesh
from ..trainer import Trainer
from .grpo import VocabSubsetReward, group_advantages, grpo_loss
from .rollout import RolloutEngine


class GRPOTrainer(Trainer):
    def __init__(self, config, reward_fn=None, **kw):
        config.data.task_type = "synthetic"
        super().__init__(config, **kw)
        rl = config.rl
        dp = mesh.get_data_parallel_world_size()
        if rl.num_prompts % dp:
            raise ValueError("rl.num_prompts must be divisible by the data-parallel size")
        self.prompts_per_replica = rl.num_prompts // dp
        self.num_seqs = self.prompts_per_replica * rl.group_size
        self.total_len = rl.prompt_len + rl.max_new_tokens
        vocab = self.model.vocab_size
        self.reward_fn = reward_fn or VocabSubsetReward(vocab, rl.reward_vocab_subset, rl.reward_seed, self.device)
        self.engine = RolloutEngine(self.model, config, max_seqs=self.num_seqs, max_seq_len=self.total_len)
        # frozen reference policy: same weights at construction time, never updated
        self.ref_model = None
        if rl.kl_beta > 0:
            from .reference_policy import frozen_copy

            self.ref_model = frozen_copy(self.model, config, self.loss_fn, self.device)
        self.prompt_gen = torch.Generator(device="cpu").manual_seed(int(rl.reward_seed) + 1000 * mesh.get_data_parallel_rank())
        self.sample_gen = None
        if self.device.type == "cuda":
            # identical sampling noise on the ranks of one TP group is not needed (each perturbs its own
            # vocabulary shard); different DP replicas must differ
            self.sample_gen = torch.Generator(device=self.device)
            self.sample_gen.manual_seed(int(config.init.seed) + 17 * mesh.get_rank())
        self.update_micro_batch = max(1, config.trainer.micro_batch_size)

    def finalize(self):
        # the decode step's captured graph holds the tensor-parallel all-reduces: it has to go before the
        # process group does, or tearing the group down waits on work that is never replayed again
        if getattr(self, "engine", None) is not None:
            self.engine.release_graph()
        super().finalize()

    def _prompts(self) -> torch.Tensor:
        rl = self.config.rl
        base = torch.randint(0, self.model.vocab_size, (self.prompts_per_replica, rl.prompt_len), generator=self.prompt_gen)
        if mesh.get_tensor_model_parallel_world_size() > 1:
            base = base.to(self.device)
            dist.broadcast(base, src=mesh.get_tensor_model_parallel_src_rank(), group=mesh.get_tensor_model_parallel_group())
        return base.repeat_interleave(rl.group_size, dim=0)

    @torch.no_grad()
    def rollout(self) -> Dict[str, torch.Tensor]:
        rl = self.config.rl
        prompts = self._prompts()
        # rollout time is measured on the device (CUDA events on the launching stream); the slowest
        # replica defines the throughput (train_step reduces it with MAX over all ranks)
        cuda = self.device.type == "cuda"
        if cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        tokens, logp_old = self.engine.generate(prompts, rl.max_new_tokens, rl.temperature, rl.top_k, rl.top_p,
                                                self.sample_gen)
        if cuda:
            e1.record()
            e1.synchronize()
            dt = e0.elapsed_time(e1) / 1e3
        else:
            dt = time.perf_counter() - t0
        generated = tokens[:, rl.prompt_len:]
        rewards = self.reward_fn(generated)
        adv = group_advantages(rewards, rl.group_size, rl.adv_eps)
        return {"tokens": tokens, "logp_old": logp_old, "rewards": rewards, "advantages": adv, "rollout_s": dt}

    def _gen_logprobs(self, model, tokens: torch.Tensor) -> torch.Tensor:
        """log-probs of the generated tokens under ``model``: [S, N]."""
        p = self.config.rl.prompt_len
        lp = model.token_logprobs(tokens[:, :-1], tokens[:, 1:])
        return lp[:, p - 1:]

    def policy_update(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        rl = self.config.rl
        tokens, logp_old, adv = batch["tokens"], batch["logp_old"], batch["advantages"]
        s = tokens.shape[0]
        mb = self.update_micro_batch
        n_mb = (s + mb - 1) // mb
        self.model.train()
        stats = {"loss": 0.0, "ratio_mean": 0.0, "kl_mean": 0.0}
        for i in range(n_mb):
            sl = slice(i * mb, min(s, (i + 1) * mb))
            tk = tokens[sl]
            with torch.no_grad():
                ref_lp = self._gen_logprobs(self.ref_model, tk) if self.ref_model is not None else None
            lp = self._gen_logprobs(self.model, tk)
            mask = torch.ones_like(lp)
            loss, st = grpo_loss(lp, logp_old[sl], ref_lp, adv[sl], mask, rl.clip_eps, rl.kl_beta)
            (loss * (tk.shape[0] / s)).backward()
            stats["loss"] += float(loss.detach()) * tk.shape[0] / s
            for k in ("ratio_mean", "kl_mean"):
                stats[k] += st[k] * tk.shape[0] / s
        grad_norm = self.optimizer.step()
        self.optimizer.zero_grad()
        self.lr_scheduler.step()
        stats["grad_norm"] = float(grad_norm) if grad_norm is not None else 0.0
        return stats

    def train_step(self, step: int):
        batch = self.rollout()
        stats = self.policy_update(batch)
        rl = self.config.rl
        gen_tokens = self.num_seqs * rl.max_new_tokens * mesh.get_data_parallel_world_size()
        stats["reward_mean"] = float(batch["rewards"].mean())
        slowest = torch.tensor([batch["rollout_s"]], dtype=torch.float64, device=self.device)
        if dist.is_initialized() and dist.get_world_size() > 1:
            slowest = slowest.float() if self.device.type == "cuda" else slowest
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        stats["rollout_s"] = float(slowest)
        stats["rollout_tokens_per_s"] = gen_tokens / max(stats["rollout_s"], 1e-9)
        return stats

    def train(self):
        steps = self.config.operation.train_steps
        for step in range(steps):
            st = self.train_step(step)
            if self.control.do_log(step) or step == steps - 1:
                self.logger.info(
                    "grpo step %d | loss %.4f | reward %.4f | kl %.5f | ratio %.4f | grad norm %.3f | rollout %.0f tok/s",
                    step + 1, st["loss"], st["reward_mean"], st["kl_mean"], st["ratio_mean"], st["grad_norm"],
                    st["rollout_tokens_per_s"])
            self.last_step = step
        return self.last_step
