"""Projection-free attention core (the projections live in the transformer layer).
``fused=True`` selects the flash kernel on CUDA (causal, GQA, optional document
boundaries); otherwise scores are materialised, which also supports arbitrary masks and
dropout. (Behavioural reference: ironcore/layers/attention.py:25-253.)"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as OF


class Attention(nn.Module):
    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, dropout: float = 0.0, fused: bool = True,
                 causal: bool = True, rotary=None):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.dropout, self.fused, self.causal = dropout, fused, causal
        self.rotary = rotary

    def forward(self, qkv: torch.Tensor, seq_len: int, pos_ids: Optional[torch.Tensor] = None,
                cu_seqlens: Optional[torch.Tensor] = None, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """qkv: packed [T, (Hq + 2 Hkv) * hd] projection output -> context [T, Hq * hd]."""
        rope = self.rotary.spec(pos_ids) if self.rotary is not None else None
        rot_dim = self.rotary.rot_dim if self.rotary is not None else None
        return OF.rope_attention(
            qkv, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, seq_len=seq_len,
            rope=rope, rot_dim=rot_dim, causal=self.causal, cu_seqlens=cu_seqlens, attn_mask=attn_mask,
            dropout_p=self.dropout, fused=self.fused, training=self.training)
