"""Python entry points of the flash attention kernels (forward and backward) operating on a
packed projection output ``qkv`` [T, (Hq + 2 Hkv) * hd] without splitting copies."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import native
from .native import call, dtype_code, ptr, stream_ptr

native.register("icb_flash_fwd", [native.P] * 5 + [native.I, native.I, native.L, native.I, native.I, native.I,
                                                   native.L, native.L, native.P, native.I, native.F, native.I,
                                                   native.P, native.P, native.F, native.P, native.I])
native.register("icb_flash_bwd", [native.P] * 11 + [native.I, native.I, native.L, native.I, native.I, native.I,
                                                    native.L, native.L, native.L, native.L, native.P, native.I,
                                                    native.F, native.I, native.P, native.P, native.F, native.P])


def available() -> bool:
    return native.available()


_MASK64 = (1 << 64) - 1
_DROPOUT_CLOCK = {}


def dropout_threshold(p: float) -> int:
    """8-bit threshold of the kernels' dropout mask: the effective drop probability is ``threshold / 256``."""
    if not p > 0:
        return 0
    return min(255, max(1, int(p * 256.0 + 0.5)))


def next_dropout_seed(device: torch.device) -> torch.Tensor:
    """The device word (int64 [1]) that selects the next attention dropout mask.

    Every device keeps a counter that starts from the global PyTorch seed and the rank and advances by one per
    call *on the device*, so that a call captured in a CUDA graph draws a new mask at every replay. The returned
    tensor is a snapshot for the backward pass."""
    clock = _DROPOUT_CLOCK.get(device)
    if clock is None:
        import torch.distributed as dist

        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        start = (torch.initial_seed() * 0x2545F4914F6CDD1D + rank * 0x9E3779B97F4A7C15) & ((1 << 62) - 1)
        clock = torch.tensor([start], dtype=torch.int64, device=device)
        _DROPOUT_CLOCK[device] = clock
    seed = clock.clone()
    clock.add_(1)
    return seed


def dropout_keep_mask(seed: int, batch: int, heads: int, max_len: int, dropout_p: float) -> torch.Tensor:
    """The keep mask [batch, heads, max_len, max_len] (bool, CPU) that the kernels derive from ``seed``: one
    splitmix64 hash per (sequence, head, query, group of 8 keys), byte ``i`` of which keeps key ``8 g + i`` when it
    is at least ``dropout_threshold(dropout_p)``. This is the definition the kernels are tested against."""
    import numpy as np

    thr = dropout_threshold(dropout_p)
    groups = (max_len + 7) // 8
    with np.errstate(over="ignore"):
        bh = np.arange(batch * heads, dtype=np.uint64).reshape(batch, heads, 1, 1)
        q = np.arange(max_len, dtype=np.uint64).reshape(1, 1, max_len, 1)
        g = np.arange(groups, dtype=np.uint64).reshape(1, 1, 1, groups)
        counter = (bh * np.uint64(max_len) + q) * np.uint64(groups) + g
        z = np.uint64(seed & _MASK64) + (counter + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
        shifts = (np.arange(8, dtype=np.uint64) * np.uint64(8)).reshape(1, 1, 1, 1, 8)
        byte = (z[..., None] >> shifts) & np.uint64(0xFF)
    keep = (byte >= np.uint64(thr)).reshape(batch, heads, max_len, groups * 8)[..., :max_len]
    return torch.from_numpy(np.ascontiguousarray(keep))


def _batch_and_len(total_tokens: int, seq_len: int, cu_seqlens: Optional[torch.Tensor]):
    if cu_seqlens is not None:
        return cu_seqlens.numel() - 1, seq_len
    return total_tokens // seq_len, seq_len


def flash_fwd(qkv: torch.Tensor, hq: int, hkv: int, hd: int, seq_len: int, *, cu_seqlens=None, causal=True,
              scale: Optional[float] = None, max_seqlen: Optional[int] = None, dropout_p: float = 0.0,
              dropout_seed: Optional[torch.Tensor] = None, wide_tiles: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (out [T, hq*hd], lse [hq, T] fp32). With ``cu_seqlens`` (int32 device tensor of
    document boundaries in the flat token stream) ``max_seqlen`` bounds the longest document
    (defaults to ``seq_len``). ``dropout_p`` > 0 drops attention probabilities inside the kernel under the mask
    that ``dropout_seed`` (int64 device tensor, see ``next_dropout_seed``) selects; the log-sum-exp is that of
    the undropped softmax."""
    if dropout_p > 0 and dropout_seed is None:
        raise ValueError("flash_fwd: dropout_p > 0 needs dropout_seed")
    t = qkv.shape[0]
    stride = qkv.stride(0)
    es = qkv.element_size()
    out = torch.empty((t, hq * hd), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((hq, t), dtype=torch.float32, device=qkv.device)
    base = qkv.data_ptr()
    batch, s = _batch_and_len(t, max_seqlen or seq_len, cu_seqlens)
    call("icb_flash_fwd", base, base + hq * hd * es, base + (hq + hkv) * hd * es, ptr(out), ptr(lse), batch, s, t,
         hq, hkv, hd, stride, stride, ptr(cu_seqlens), 1 if causal else 0, float(scale if scale else hd ** -0.5),
         dtype_code(qkv.dtype), ptr(native.status_tensor(qkv.device)), stream_ptr(), float(dropout_p),
         ptr(dropout_seed), 1 if wide_tiles else 0)
    return out, lse


def flash_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, hq: int, hkv: int, hd: int,
              seq_len: int, *, cu_seqlens=None, causal=True, scale: Optional[float] = None,
              max_seqlen: Optional[int] = None, dropout_p: float = 0.0,
              dropout_seed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Returns dqkv with the packed layout of ``qkv``. ``dropout_p`` / ``dropout_seed`` are the forward's."""
    if dropout_p > 0 and dropout_seed is None:
        raise ValueError("flash_bwd: dropout_p > 0 needs dropout_seed")
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
         stream_ptr(), float(dropout_p), ptr(dropout_seed))
    return dqkv
