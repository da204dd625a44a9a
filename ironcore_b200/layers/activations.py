"""Activation registry. Plain: relu, gelu, gelu_tanh (a.k.a. gelu_new), silu. Gated (applied to
[f | g] halves of the up projection): swiglu = silu(f)*g, geglu = gelu_tanh(f)*g,
geglu_erf, reglu, glu = f*sigmoid(g).
(Behavioural reference: ironcore/layers/activations/activations.py:15-60; the gated forms use
the published definitions.)"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as OF

_ALIASES = {"gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "swish": "silu", "siglu": "glu"}


def canonical_activation(name: str) -> str:
    name = name.lower()
    return _ALIASES.get(name, name)


def is_glu(name: str) -> bool:
    return OF.is_gated(canonical_activation(name))


class Activation(nn.Module):
    def __init__(self, name: str):
        super().__init__()
        self.name = canonical_activation(name)
        self.gated = OF.is_gated(self.name)

    def forward(self, x: torch.Tensor, row_limit=None) -> torch.Tensor:
        return OF.activation(x, self.name, row_limit)

    def extra_repr(self):
        return self.name


def get_activation(name: str, dim: int = 0) -> Activation:
    return Activation(name)
