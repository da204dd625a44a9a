"""LayerNorm / RMSNorm modules backed by the fused norm kernel (optionally fused with the
residual add that precedes the norm). Parameter path is ``<name>.layernorm.weight|bias``.
(Behavioural reference: ironcore/layers/layernorm/*.py.)"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as OF


class _NormParams(nn.Module):
    def __init__(self, dim: int, bias: bool, init_weight: float, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.full((dim,), init_weight, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if bias else None
        # replicated over TP but sees different tokens per rank under sequence parallelism
        self.weight.sp_replicated = True
        if self.bias is not None:
            self.bias.sp_replicated = True


class Norm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, rms: bool = False, bias: bool = True, weight_offset: float = 0.0,
                 dtype=None, device=None):
        super().__init__()
        self.dim, self.eps, self.rms, self.weight_offset = dim, eps, rms, weight_offset
        self.layernorm = _NormParams(dim, bias and not rms, 1.0 - weight_offset, dtype, device)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, return_sum: bool = False,
                out: Optional[torch.Tensor] = None):
        y, h = OF.norm(x, self.layernorm.weight, self.layernorm.bias, self.eps, self.rms, residual=residual,
                       w_offset=self.weight_offset, out=out)
        return (y, h) if return_sum else y


class FusedLayerNorm(Norm):
    def __init__(self, dim, eps=1e-5, bias=True, **kw):
        super().__init__(dim, eps, rms=False, bias=bias, **kw)


class FusedRMSNorm(Norm):
    def __init__(self, dim, eps=1e-5, **kw):
        kw.pop("bias", None)
        super().__init__(dim, eps, rms=True, bias=False, **kw)


def get_norm(config, dtype=None, device=None) -> Norm:
    m = config.model
    rms = m.ln_type == "rmsnorm"
    return Norm(m.d_model, m.ln_eps, rms=rms, bias=not m.no_bias, weight_offset=float(m.norm_weight_offset or 0.0),
                dtype=dtype, device=device)
