"""Paged-cache ops: native kernels on CUDA, PyTorch restatements elsewhere (oracle / CPU path)."""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import native
from ..ops.native import call, dtype_code, ptr, stream_ptr

P, I, L, F = native.P, native.I, native.L, native.F
native.register("icb_kv_append", [P, P, P, P, P, I, I, L, L, P])
native.register("icb_paged_decode", [P, L, P, P, P, P, P, P, I, I, I, I, I, I, F, I, P, P, I])
_SMS = None


def _decode_splits(num_seqs: int, hkv: int, max_tokens: int) -> int:
    """Context ranges per (sequence, kv head) for the tensor-core decode kernel: enough CTAs for two per SM,
    at least four 16-token steps per range."""
    global _SMS
    if _SMS is None:
        _SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    want = -(-2 * _SMS // max(1, num_seqs * hkv))
    return max(1, min(want, 8, max(1, max_tokens // 64)))
native.register("icb_grpo_loss", [P, P, P, P, P, P, P, P, P, L, F, F, P])


def kv_append(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor):
    """k, v: [T, hkv*hd] (row views with arbitrary pitch); caches [blocks, bs, hkv, hd]; slots int64 [T]."""
    t, row = k.shape
    if k.is_cuda and k.dtype in (torch.bfloat16, torch.float16):
        call("icb_kv_append", ptr(k), ptr(v), ptr(k_cache), ptr(v_cache), ptr(slots), t, row, k.stride(0), v.stride(0),
             stream_ptr())
        return
    kc = k_cache.view(-1, row)
    vc = v_cache.view(-1, row)
    ok = slots >= 0
    kc[slots[ok]] = k[ok]
    vc[slots[ok]] = v[ok]


def paged_decode_reference(q, k_cache, v_cache, block_table, seq_lens, hq, hkv, hd, scale):
    s = q.shape[0]
    bs = k_cache.shape[1]
    out = torch.zeros((s, hq * hd), dtype=q.dtype, device=q.device)
    g = hq // hkv
    for i in range(s):
        n = int(seq_lens[i])
        if n == 0:
            continue
        pages = (n + bs - 1) // bs
        blocks = block_table[i, :pages].long()
        k = k_cache[blocks].reshape(-1, hkv, hd)[:n].float()
        v = v_cache[blocks].reshape(-1, hkv, hd)[:n].float()
        qi = q[i].view(hq, hd).float()
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        sc = torch.einsum("hd,nhd->hn", qi, k) * scale
        p = torch.softmax(sc, dim=-1)
        out[i] = torch.einsum("hn,nhd->hd", p, v).reshape(-1).to(q.dtype)
    return out


def paged_decode(q: torch.Tensor, k_cache, v_cache, block_table, seq_lens, hq: int, hkv: int, hd: int,
                 scale: Optional[float] = None) -> torch.Tensor:
    """q: [S, hq*hd] (row view, any pitch) -> [S, hq*hd]: attention of one token per sequence over its pages."""
    scale = scale if scale is not None else hd ** -0.5
    s = q.shape[0]
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and hd in (64, 128) and hq // hkv <= 8:
        out = torch.empty((s, hq * hd), dtype=q.dtype, device=q.device)
        scratch, nsplit = None, 0
        if hd == 128 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0:
            # tensor-core kernel (mma.sync over the GQA group), the context split over several CTAs
            nsplit = _decode_splits(s, hkv, block_table.shape[1] * k_cache.shape[1])
            scratch = torch.empty(max(1, s * hq * nsplit * (hd + 2)), dtype=torch.float32, device=q.device)
        call("icb_paged_decode", ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache), ptr(block_table), ptr(seq_lens),
             ptr(out), None, s, hq, hkv, hd, k_cache.shape[1], block_table.shape[1], float(scale),
             dtype_code(q.dtype), stream_ptr(), ptr(scratch), int(nsplit))
        return out
    return paged_decode_reference(q, k_cache, v_cache, block_table, seq_lens, hq, hkv, hd, scale)


class _GrpoLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, logp_old, logp_ref, adv, mask, eps, beta):
        n = logp.numel()
        loss = torch.empty_like(logp)
        dlogp = torch.empty_like(logp)
        ratio = torch.empty_like(logp)
        kl = torch.empty_like(logp)
        call("icb_grpo_loss", ptr(logp), ptr(logp_old), ptr(logp_ref), ptr(adv), ptr(mask), ptr(loss), ptr(dlogp),
             ptr(ratio), ptr(kl), n, float(eps), float(beta), stream_ptr())
        ctx.save_for_backward(dlogp)
        ctx.mark_non_differentiable(ratio, kl)
        return loss, ratio, kl

    @staticmethod
    def backward(ctx, gloss, _gr, _gk):
        (dlogp,) = ctx.saved_tensors
        return gloss * dlogp, None, None, None, None, None, None


def grpo_token_loss(logp, logp_old, logp_ref, adv, mask, eps: float, beta: float):
    """Per-token GRPO loss (PPO-clip + beta * k3 KL). All inputs fp32 [N]; returns (loss, ratio, kl)."""
    if logp.is_cuda:
        f = lambda t: None if t is None else t.contiguous().float()
        return _GrpoLoss.apply(f(logp), f(logp_old), f(logp_ref), f(adv), f(mask), eps, beta)
    ratio = torch.exp(logp - logp_old)
    pg = -torch.minimum(ratio * adv, ratio.clamp(1 - eps, 1 + eps) * adv)
    if logp_ref is not None:
        delta = logp_ref - logp
        kl = torch.exp(delta) - delta - 1
    else:
        kl = torch.zeros_like(logp)
    return mask * (pg + beta * kl), ratio.detach(), kl.detach()
