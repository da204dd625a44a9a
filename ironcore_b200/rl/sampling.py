"""Token sampling from (vocab-sharded) logits: temperature, top-k, top-p; exact sampling through
the Gumbel-max trick so that a tensor-parallel vocabulary never has to be gathered — every rank
perturbs its own shard and the arg-max is combined across ranks with two small all-gathers."""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def _filter_top_k_top_p(logits: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    if top_k and top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.shape[-1]), dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        sorted_logits, idx = torch.sort(logits, dim=-1, descending=True)
        probs = torch.softmax(sorted_logits, dim=-1)
        cum = probs.cumsum(-1)
        drop = cum - probs > top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, sorted_logits)
    return logits


def sample_tokens(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                  generator: Optional[torch.Generator] = None, vocab_start: int = 0, vocab_valid: Optional[int] = None,
                  group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits [S, V_local] -> (token ids [S] int64 in the global vocabulary, log-prob of each under
    the *unfiltered* temperature-scaled distribution, fp32)."""
    lf = logits.float()
    v_local = lf.shape[-1]
    if vocab_valid is not None and vocab_valid < v_local:
        lf[:, vocab_valid:] = float("-inf")
    sharded = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
    if (top_k and top_k > 0) or (top_p is not None and top_p < 1.0):
        if sharded:
            parts = [torch.empty_like(lf) for _ in range(dist.get_world_size(group))]
            dist.all_gather(parts, lf.contiguous(), group=group)
            lf = torch.cat(parts, dim=-1)
            vocab_start, sharded = 0, False
    if temperature <= 0:
        scaled = lf
        pert = lf
    else:
        scaled = lf / temperature
        filt = _filter_top_k_top_p(scaled, top_k, top_p)
        u = torch.rand(filt.shape, device=filt.device, generator=generator).clamp_(1e-20, 1.0)
        pert = filt - torch.log(-torch.log(u))
    best_val, best_idx = pert.max(dim=-1)
    lmax = scaled.max(dim=-1).values
    if sharded:
        world = dist.get_world_size(group)
        vals = [torch.empty_like(best_val) for _ in range(world)]
        idxs = [torch.empty_like(best_idx) for _ in range(world)]
        dist.all_gather(vals, best_val.contiguous(), group=group)
        dist.all_gather(idxs, (best_idx + vocab_start).contiguous(), group=group)
        winner = torch.stack(vals).argmax(dim=0, keepdim=True)
        token = torch.stack(idxs).gather(0, winner).squeeze(0)
        gmax = lmax.clone()
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        sumexp = torch.exp(scaled - gmax[:, None]).sum(-1)
        dist.all_reduce(sumexp, group=group)
        local = token - vocab_start
        mine = (local >= 0) & (local < v_local)
        tl = scaled.gather(1, local.clamp(0, v_local - 1)[:, None]).squeeze(1) * mine.float()
        dist.all_reduce(tl, group=group)
        logp = tl - (gmax + torch.log(sumexp))
    else:
        token = best_idx + vocab_start
        lse = torch.logsumexp(scaled, dim=-1)
        logp = scaled.gather(1, best_idx[:, None]).squeeze(1) - lse
    return token, logp
