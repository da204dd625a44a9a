"""Token sampling from (vocab-sharded) logits: temperature, top-k, top-p; exact sampling through
the Gumbel-max trick so that a tensor-parallel vocabulary never has to be gathered — every rank
perturbs its own shard and the arg-max is combined across ranks with two small all-gathers.

On CUDA, plain temperature sampling (no top-k / top-p filter) is one kernel per step
(``csrc/sampling.cu``): a single pass over each row produces the sample and the row's softmax
statistics; nothing of size ``[S, V]`` is written. The PyTorch path below serves the filters, CPU
tensors and greedy decoding, and is the oracle of the kernel."""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import native

native.register("icb_sample_gumbel", [native.P, native.L, native.I, native.I, native.I, native.F,
                                      native.C.c_ulonglong, native.C.c_ulonglong, native.L, native.I, native.P,
                                      native.P, native.P, native.P])
native.register("icb_sample_parts", [native.I, native.I])
_DRAWS = {}


def _next_draw(generator) -> tuple:
    """(seed, draw counter) of the noise stream of ``generator`` (one counter per generator object)."""
    seed = int(generator.initial_seed()) if generator is not None else int(torch.initial_seed())
    key = id(generator) if generator is not None else None
    draw = _DRAWS.get(key, 0)
    _DRAWS[key] = draw + 1
    return seed & (2 ** 64 - 1), draw


def _sample_native(logits: torch.Tensor, temperature: float, generator, vocab_start: int, vocab_valid: int, group):
    """One kernel per step; see the module docstring. Returns (token, logp)."""
    s, v = logits.shape
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    stats = torch.empty((s, 4), dtype=torch.float32, device=logits.device)
    index = torch.empty(s, dtype=torch.int32, device=logits.device)
    seed, draw = _next_draw(generator)
    parts = native.query("icb_sample_parts", int(s), int(v))
    scratch = torch.empty(s * parts * 5, dtype=torch.float32, device=logits.device) if parts > 1 else None
    native.call("icb_sample_gumbel", native.ptr(logits), int(logits.stride(0)), int(s), int(v), int(vocab_valid),
                float(temperature), seed, draw, int(vocab_start), native.dtype_code(logits.dtype), native.ptr(stats),
                native.ptr(index), native.ptr(scratch), native.stream_ptr())
    best, best_x, mx, sm = stats.unbind(1)
    if group is None:
        return index.long() + vocab_start, best_x - (mx + torch.log(sm))
    world = dist.get_world_size(group)
    all_stats = torch.empty((world, s, 4), dtype=torch.float32, device=logits.device)
    all_index = torch.empty((world, s), dtype=torch.int32, device=logits.device)
    dist.all_gather_into_tensor(all_stats, stats, group=group)
    dist.all_gather_into_tensor(all_index, index, group=group)
    starts = torch.arange(world, device=logits.device, dtype=torch.int64)[:, None] * v
    winner = all_stats[..., 0].argmax(dim=0, keepdim=True)
    token = (all_index.long() + starts).gather(0, winner).squeeze(0)
    chosen = all_stats[..., 1].gather(0, winner).squeeze(0)
    gmax = all_stats[..., 2].max(dim=0).values
    total = (all_stats[..., 3] * torch.exp(all_stats[..., 2] - gmax)).sum(0)
    return token, chosen - (gmax + torch.log(total))


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
    sharded = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
    filtered = (top_k and top_k > 0) or (top_p is not None and top_p < 1.0)
    if logits.is_cuda and logits.dim() == 2 and temperature > 0 and not filtered \
            and logits.dtype in (torch.bfloat16, torch.float16, torch.float32):
        valid = logits.shape[-1] if vocab_valid is None else vocab_valid
        return _sample_native(logits, temperature, generator, vocab_start, valid, group if sharded else None)
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
