"""fc1 -> ReLU -> fc2 stack for plumbing tests (``model: dummy``).
(Behavioural reference: ironcore/models/dummy.py:18-65.)"""

from __future__ import annotations

import torch.nn as nn
import torch.nn.functional as F


class DummyModel(nn.Module):
    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        m = config.model
        self.blocks = nn.ModuleList()
        for _ in range(m.num_layers):
            self.blocks.append(nn.ModuleDict({
                "fc1": nn.Linear(m.d_model, m.d_ffn, dtype=dtype, device=device),
                "fc2": nn.Linear(m.d_ffn, m.d_model, dtype=dtype, device=device),
            }))

    def forward(self, x, seq_len=None, pos_ids=None, cu_seqlens=None, attn_mask=None):
        for blk in self.blocks:
            x = x + blk["fc2"](F.relu(blk["fc1"](x)))
        return x, None
