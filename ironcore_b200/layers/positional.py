"""Positional embeddings: rotary (applied inside the fused attention op), fixed sinusoidal
table and the learned absolute table (owned by the embedding layer).
(Behavioural reference: ironcore/layers/positional_embedding/rotary.py:15-83 — with the
rotation taken along the *sequence* position — and absolute.py:17-35.)"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import reference


class RotaryPositionalEmbedding(nn.Module):
    """Holds the rotary hyper-parameters and exposes the op-level description consumed by
    :func:`ironcore_b200.ops.functional.rope_attention`; ``forward`` rotates a
    [B, S, H, hd] tensor directly (used by tests, the paged-decode path and tooling)."""

    def __init__(self, head_dim: int, base: float = 10000.0, scaling_factor: float = 1.0, offset: int = 0,
                 interleaved: bool = True, rotary_fraction: float = 1.0):
        super().__init__()
        self.head_dim = head_dim
        self.base = float(base)
        self.scaling_factor = float(scaling_factor)
        self.offset = int(offset)
        self.interleaved = bool(interleaved)
        rot = int(head_dim * rotary_fraction)
        self.rot_dim = rot - (rot % 2)
        theta = self.base ** (-torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim)
        self.register_buffer("theta", theta, persistent=True)

    def spec(self, pos_ids: Optional[torch.Tensor] = None):
        return (self.base, self.scaling_factor, self.offset, self.interleaved, pos_ids)

    def forward(self, x: torch.Tensor, pos_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, s = x.shape[0], x.shape[1]
        if pos_ids is None:
            pos_ids = torch.arange(s, device=x.device).expand(b, s)
        if self.rot_dim == self.head_dim:
            return reference.rope_reference(x, pos_ids, self.base, self.scaling_factor, self.offset, self.interleaved)
        rot = reference.rope_reference(x[..., :self.rot_dim], pos_ids, self.base, self.scaling_factor, self.offset,
                                       self.interleaved)
        return torch.cat([rot, x[..., self.rot_dim:]], dim=-1)


class SinusoidalPositionalEmbedding(nn.Module):
    def __init__(self, max_len: int, dim: int):
        super().__init__()
        pos = torch.arange(max_len, dtype=torch.float32)[:, None]
        div = torch.exp(torch.arange(0, dim, 2, dtype=torch.float32) * (-math.log(10000.0) / dim))
        table = torch.zeros(max_len, dim)
        table[:, 0::2] = torch.sin(pos * div)
        table[:, 1::2] = torch.cos(pos * div)[:, : dim // 2]
        self.register_buffer("table", table, persistent=False)

    def forward(self, pos_ids: torch.Tensor) -> torch.Tensor:
        return self.table[pos_ids]
