"""Attention core with the reference's call convention: built from the configuration, called with separate
query / key / value tensors (reference: ironcore/layers/attention.py:25-253)."""

from __future__ import annotations

import torch
from torch import nn

from ironcore_b200.layers.module import BaseModule
from ironcore_b200.ops import functional as OF


class Attention(BaseModule):
    """``forward(query [b, s, hn, hd], key [b, s, gn, hd], value [b, s, gn, hd], attention_mask) -> [b, s, hn * hd]``.

    With ``trainer.use_flash_attn`` the flash kernel runs (always causal; the mask is not read, as in the
    reference's flash path). Otherwise the scores are materialised: positions where ``attention_mask == 0`` are
    masked out, and without a mask the attention is bidirectional. Rotary embedding, if any, has already been
    applied by the caller."""

    def __init__(self, config):
        super().__init__(config)
        m, tp = config.model, config.trainer.tensor_model_parallel_size
        self.num_attention_heads = m.num_attention_heads
        self.tensor_model_parallel_size = tp
        self.head_dimension = m.head_dim or m.d_model // m.num_attention_heads
        self.num_local_attention_heads = m.num_attention_heads // tp
        self.num_local_attention_groups = m.num_attention_groups // tp
        self.softmax = nn.Softmax(dim=-1)
        self.attn_dropout = nn.Dropout(m.dropout_attn)
        self.scale_factor = self.head_dimension ** 0.5

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, attention_mask=None) -> torch.Tensor:
        b, s, hq, hd = query.shape
        hkv = key.shape[2]
        if key.shape[1] != s:
            raise ValueError("query and key / value need the same sequence length (self attention)")
        qkv = torch.cat([query.reshape(b * s, hq * hd), key.reshape(b * s, hkv * hd), value.reshape(b * s, hkv * hd)],
                        dim=-1)
        flash = bool(self.config.trainer.use_flash_attn)
        mask = None
        if not flash and attention_mask is not None:
            mask = attention_mask != 0
        out = OF.rope_attention(qkv, num_heads=hq, num_kv_heads=hkv, head_dim=hd, seq_len=s, rope=None, causal=flash,
                                scale=1.0 / self.scale_factor, attn_mask=mask,
                                dropout_p=float(self.config.model.dropout_attn), fused=flash, training=self.training)
        return out.reshape(b, s, hq * hd)
