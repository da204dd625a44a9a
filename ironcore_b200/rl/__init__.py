"""Rollouts and RL: block KV cache, paged decode attention, sampling, rollout engine, GRPO; DPO on preference
pairs (``rl.dpo``: imported on demand, it pulls in the trainer)."""

from .grpo import VocabSubsetReward, group_advantages, grpo_loss
from .kv_cache import BlockKVCache
from .rollout import RolloutEngine
from .sampling import sample_tokens

__all__ = ["BlockKVCache", "RolloutEngine", "VocabSubsetReward", "group_advantages", "grpo_loss", "sample_tokens"]
