"""Plain PyTorch restatements of every native op. They are the CPU execution path,
the numerical oracle for the GPU tests, and the semantics definition of each op."""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def act_reference(x: torch.Tensor, name: str) -> torch.Tensor:
    if name == "relu":
        return F.relu(x)
    if name == "gelu":
        return F.gelu(x)
    if name == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if name == "silu":
        return F.silu(x)
    if name == "sigmoid":
        return torch.sigmoid(x)
    raise ValueError(f"unknown activation {name}")


def glu_reference(x: torch.Tensor, name: str) -> torch.Tensor:
    """Gated activations on x = [f | g] (halves of the last dim)."""
    f, g = x.chunk(2, dim=-1)
    if name == "swiglu":
        return F.silu(f) * g
    if name == "geglu":
        return F.gelu(f, approximate="tanh") * g
    if name == "geglu_erf":
        return F.gelu(f) * g
    if name == "reglu":
        return F.relu(f) * g
    if name == "glu":
        return f * torch.sigmoid(g)
    raise ValueError(f"unknown gated activation {name}")


def rms_norm_reference(x, weight, eps: float, w_offset: float = 0.0):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (weight.float() + w_offset)
    return y.to(x.dtype)


def layer_norm_reference(x, weight, bias, eps: float):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def rope_angles(positions: torch.Tensor, head_dim: int, base: float, scale: float = 1.0, offset: int = 0):
    inv = base ** (-torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim)
    ang = (positions.float() + offset)[..., None] * scale * inv
    return ang.cos(), ang.sin()


def rope_reference(x: torch.Tensor, positions: torch.Tensor, base: float, scale: float = 1.0, offset: int = 0,
                   interleaved: bool = True, inverse: bool = False) -> torch.Tensor:
    """x: [..., T, H, hd]; positions: [..., T]. Rotation along the sequence position."""
    hd = x.shape[-1]
    c, s = rope_angles(positions, hd, base, scale, offset)
    c, s = c.unsqueeze(-2), s.unsqueeze(-2)
    if inverse:
        s = -s
    xf = x.float()
    if interleaved:
        x0, x1 = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1).flatten(-2)
    else:
        x0, x1 = xf[..., : hd // 2], xf[..., hd // 2:]
        out = torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1)
    return out.to(x.dtype)


def attention_reference(q, k, v, causal: bool = True, scale: Optional[float] = None,
                        cu_seqlens: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None):
    """q: [B, S, Hq, hd], k/v: [B, S, Hkv, hd] -> [B, S, Hq, hd]. fp32 softmax, GQA by head repetition."""
    b, s, hq, hd = q.shape
    hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2)
    vf = v.float().transpose(1, 2)
    if hkv != hq:
        rep = hq // hkv
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    scores = qf @ kf.transpose(-1, -2) * scale
    sk = kf.shape[2]
    if causal:
        cm = torch.ones(s, sk, dtype=torch.bool, device=q.device).tril(diagonal=sk - s)
        scores = scores.masked_fill(~cm, float("-inf"))
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    out = p @ vf
    return out.transpose(1, 2).to(q.dtype)
