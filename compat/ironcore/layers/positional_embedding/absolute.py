"""Absolute positional embeddings (reference: ironcore/layers/positional_embedding/absolute.py:17-35)."""

import torch

from ironcore_b200.layers.positional import SinusoidalPositionalEmbedding


class PositionalEncoding(SinusoidalPositionalEmbedding):
    """``forward(x [b, s, d]) -> x + table[:s]`` with the fixed sine / cosine table, indexed by the position
    in the sequence (dimension -2)."""

    def __init__(self, d_model: int, max_len: int = 4096):
        super().__init__(max_len, d_model)
        self.d_model, self.max_len = d_model, max_len

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # pylint: disable=arguments-differ
        pos = torch.arange(x.shape[-2], device=x.device)
        return x + super().forward(pos).to(x.dtype)
