"""Python entry points of the flash attention kernels (forward and backward) operating on a
packed projection output ``qkv`` [T, (Hq + 2 Hkv) * hd] without splitting copies."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import native
from .native import call, dtype_code, ptr, stream_ptr

native.register("icb_flash_fwd", [native.P] * 5 + [native.I, native.I, native.L, native.I, native.I, native.I,
                                                   native.L, native.L, native.P, native.I, native.F, native.I,
                                                   native.P, native.P])
native.register("icb_flash_bwd", [native.P] * 11 + [native.I, native.I, native.L, native.I, native.I, native.I,
                                                    native.L, native.L, native.L, native.L, native.P, native.I,
                                                    native.F, native.I, native.P, native.P])


def available() -> bool:
    return native.available()


def _batch_and_len(total_tokens: int, seq_len: int, cu_seqlens: Optional[torch.Tensor]):
    if cu_seqlens is not None:
        return cu_seqlens.numel() - 1, seq_len
    return total_tokens // seq_len, seq_len


def flash_fwd(qkv: torch.Tensor, hq: int, hkv: int, hd: int, seq_len: int, *, cu_seqlens=None, causal=True,
              scale: Optional[float] = None, max_seqlen: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (out [T, hq*hd], lse [hq, T] fp32). With ``cu_seqlens`` (int32 device tensor of
    document boundaries in the flat token stream) ``max_seqlen`` bounds the longest document
    (defaults to ``seq_len``)."""
    t = qkv.shape[0]
    stride = qkv.stride(0)
    es = qkv.element_size()
    out = torch.empty((t, hq * hd), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((hq, t), dtype=torch.float32, device=qkv.device)
    base = qkv.data_ptr()
    batch, s = _batch_and_len(t, max_seqlen or seq_len, cu_seqlens)
    call("icb_flash_fwd", base, base + hq * hd * es, base + (hq + hkv) * hd * es, ptr(out), ptr(lse), batch, s, t,
         hq, hkv, hd, stride, stride, ptr(cu_seqlens), 1 if causal else 0, float(scale if scale else hd ** -0.5),
         dtype_code(qkv.dtype), ptr(native.status_tensor(qkv.device)), stream_ptr())
    return out, lse


def flash_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, hq: int, hkv: int, hd: int,
              seq_len: int, *, cu_seqlens=None, causal=True, scale: Optional[float] = None,
              max_seqlen: Optional[int] = None) -> torch.Tensor:
    """Returns dqkv with the packed layout of ``qkv``."""
    t = qkv.shape[0]
    stride = qkv.stride(0)
    es = qkv.element_size()
    dqkv = torch.empty((t, (hq + 2 * hkv) * hd), dtype=qkv.dtype, device=qkv.device)
    delta = torch.empty((hq, t), dtype=torch.float32, device=qkv.device)
    dq_acc = torch.empty((t, hq * hd), dtype=torch.float32, device=qkv.device)
    base, dbase = qkv.data_ptr(), dqkv.data_ptr()
    dstride = dqkv.stride(0)
    batch, s = _batch_and_len(t, max_seqlen or seq_len, cu_seqlens)
    call("icb_flash_bwd", ptr(dout), base, base + hq * hd * es, base + (hq + hkv) * hd * es, ptr(out), ptr(lse),
         dbase, dbase + hq * hd * es, dbase + (hq + hkv) * hd * es, ptr(delta), ptr(dq_acc), batch, s, t, hq, hkv, hd,
         stride, stride, dstride, dstride, ptr(cu_seqlens), 1 if causal else 0,
         float(scale if scale else hd ** -0.5), dtype_code(qkv.dtype), ptr(native.status_tensor(qkv.device)),
         stream_ptr())
    return dqkv
