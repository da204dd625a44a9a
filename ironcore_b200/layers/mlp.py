"""Feed-forward block: column-parallel up projection (gate|up fused for gated activations,
each half sharded separately), activation, row-parallel down projection whose epilogue
adds the residual. (Behavioural reference: ironcore/layers/mlp.py:19-54.)"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from .activations import Activation


class MLP(nn.Module):
    def __init__(self, d_model: int, d_ffn: int, activation: str, bias: bool = True, dropout: float = 0.0,
                 dtype=None, device=None, tp_group="default"):
        super().__init__()
        self.activation = Activation(activation)
        mult = 2 if self.activation.gated else 1
        self.up_proj = ColumnParallelLinear(d_model, d_ffn * mult, bias=bias, concatenated_weights=mult, dtype=dtype,
                                            device=device, tp_group=tp_group)
        self.down_proj = RowParallelLinear(d_ffn, d_model, bias=bias, input_is_parallel=True, dtype=dtype,
                                           device=device, tp_group=tp_group)
        self.dropout = dropout

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, up_out: Optional[torch.Tensor] = None,
                next_norm=None, next_consumer=None):
        """``up_out``: the up projection of ``x`` when the caller already computed it (fused norm boundary).
        ``next_norm`` / ``next_consumer``: the norm and column-parallel linear that follow this block; when
        given the result is ``(out, y_next)`` with ``y_next = next_consumer(next_norm(out))`` computed inside
        the fused boundary kernels, or ``(out, None)`` when that is not possible."""
        h = self.activation(self.up_proj(x) if up_out is None else up_out)
        if self.dropout > 0 and self.training:
            y = F.dropout(self.down_proj(h), self.dropout, True)
            y = y if residual is None else y + residual
            return (y, None) if next_norm is not None else y
        if next_norm is not None:
            if self.down_proj.can_fuse_norm(h, next_norm, next_consumer):
                return self.down_proj.forward_norm_linear(h, residual, next_norm, next_consumer)
            return self.down_proj(h, residual=residual), None
        return self.down_proj(h, residual=residual)
