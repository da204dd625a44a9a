"""Normalisation layers (reference: ironcore/layers/layernorm/)."""

from ironcore_b200.layers.norm import FusedLayerNorm, FusedRMSNorm, Norm, get_norm  # noqa: F401
