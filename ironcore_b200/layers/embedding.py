"""Token embedding (vocab-parallel) + optional learned position table + dropout.
Output is token-major [B*S, D] (a token shard under sequence parallelism).
(Behavioural reference: ironcore/layers/embedding.py:9-50.)"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel.tensor_parallel import VocabParallelEmbedding


class LanguageModelEmbedding(nn.Module):
    def __init__(self, padded_vocab: int, vocab_size: int, d_model: int, max_positions: int, learned_positions: bool,
                 dropout: float = 0.0, scale: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.word_embeddings = VocabParallelEmbedding(padded_vocab, d_model, padding_start_idx=vocab_size,
                                                      dtype=dtype, device=device)
        self.position_embedding = nn.Embedding(max_positions, d_model, dtype=dtype, device=device) \
            if learned_positions else None
        self.dropout = dropout
        self.scale = scale

    def forward(self, ids: torch.Tensor, pos_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        pt = self.position_embedding.weight if self.position_embedding is not None else None
        if self.scale is not None and pt is not None:
            raise ValueError("embedding scale with a learned position table is not supported")
        x = self.word_embeddings(ids, pos_table=pt, pos_ids=pos_ids)
        if self.scale is not None:
            x = x * self.scale
        if self.dropout > 0 and self.training:
            x = F.dropout(x, self.dropout, True)
        return x
