"""Normalisation layers (reference: ironcore/layers/layernorm/__init__.py:15-26)."""

from ironcore_b200.layers.norm import FusedLayerNorm, FusedRMSNorm, Norm  # noqa: F401

from .fused_layer_norm import LayerNorm
from .fused_rms_norm import RmsNorm


def get_norm(config):
    ln_type = config.model.ln_type.lower()
    if ln_type == "layernorm":
        return LayerNorm(config)
    if ln_type == "rmsnorm":
        return RmsNorm(config)
    raise NotImplementedError(f"{config.model.ln_type} is not supported")
