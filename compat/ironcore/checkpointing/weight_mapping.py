"""Parameter-name mapping between the ironcore and the HuggingFace layouts with the reference's mapper API
(reference: ironcore/checkpointing/weight_mapping.py:35-330).

``WeightMapper(architecture, num_layers).hf_to_ironcore(...)`` produces the *mapper dialect* the reference documents
for this API: attention tensors under ``model.layers.N.self_attention.{linear_q,linear_kv,output}``, norm tensors as
``<norm>.weight`` and every linear weight as ``[out, in]``. ``ironcore_b200`` models use the live parameter names
(``model.layers.N.linear_q``, ``<norm>.layernorm.weight``) and ``[in, out]`` weights; ``to_live`` / ``from_live``
convert between the two, and ``ironcore_to_hf`` accepts either."""

from __future__ import annotations

import re
from typing import Dict

import torch

from ironcore_b200.checkpoint import hf_interop as _hf
from ironcore_b200.checkpoint.hf_interop import _ALIASES as ARCHITECTURE_ALIASES  # noqa: F401
from ironcore_b200.checkpoint.hf_interop import Architecture, detect_architecture  # noqa: F401

get_architecture = detect_architecture

_LIVE_TO_DIALECT = (("linear_q.", "self_attention.linear_q."), ("linear_kv.", "self_attention.linear_kv."),
                    ("attn_output.", "self_attention.output."))
_LINEAR = re.compile(r"(linear_q|linear_kv|attn_output|self_attention\.output|up_proj|down_proj|output_layer)\.weight$")


def from_live(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Live ``ironcore_b200`` names and ``[in, out]`` weights -> the mapper dialect."""
    out = {}
    for k, v in sd.items():
        if _LINEAR.search(k) and v.dim() == 2:
            v = v.t().contiguous()
        k = k.replace(".layernorm.", ".")
        m = re.match(r"(model\.layers\.\d+\.)(.*)$", k)
        if m:
            rest = m.group(2)
            for live, dia in _LIVE_TO_DIALECT:
                if rest.startswith(live):
                    rest = dia + rest[len(live):]
                    break
            k = m.group(1) + rest
        out[k] = v
    return out


def to_live(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The mapper dialect -> live ``ironcore_b200`` names and ``[in, out]`` weights. A dictionary that already uses
    the live names (no ``self_attention`` entries) is returned unchanged."""
    if not any(".self_attention." in k for k in sd):
        return dict(sd)
    out = {}
    for k, v in sd.items():
        k = k.replace(".self_attention.output.", ".attn_output.").replace(".self_attention.", ".")
        if ".layernorm.layernorm." not in k:
            k = re.sub(r"layernorm\.(weight|bias)$", r"layernorm.layernorm.\1", k)
        if _LINEAR.search(k) and v.dim() == 2:
            v = v.t().contiguous()
        out[k] = v
    return out


class WeightMapper(_hf.WeightMapper):
    """``WeightMapper(architecture, num_layers)``. Without head counts no rotary permutation is applied (names and
    layouts only, as in the reference); pass ``num_heads`` / ``num_kv_heads`` / ``head_dim`` for a
    forward-equivalent import of rotary models."""

    def __init__(self, architecture: Architecture, num_layers: int, num_heads: int = None, num_kv_heads: int = None,
                 head_dim: int = None, **kw):
        if num_heads is None or head_dim is None:
            kw["interleaved_rope"] = False
            num_heads, num_kv_heads, head_dim = 0, 0, 0
        super().__init__(architecture, num_layers, num_heads, num_kv_heads or num_heads, head_dim, **kw)
        self.architecture, self.num_layers = architecture, num_layers

    def hf_to_ironcore(self, hf_state_dict: Dict[str, torch.Tensor], strict: bool = True) -> Dict[str, torch.Tensor]:
        try:
            return from_live(self.hf_to_native(hf_state_dict))
        except KeyError as e:
            raise KeyError(f"HuggingFace state dict lacks {e} (strict={strict}: every tensor of the "
                           f"{self.num_layers}-layer model is needed either way)") from e

    def ironcore_to_hf(self, ironcore_state_dict: Dict[str, torch.Tensor], strict: bool = True) -> Dict[str, torch.Tensor]:
        return self.native_to_hf(to_live(ironcore_state_dict))
