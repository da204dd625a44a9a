"""LayerNorm built from the configuration (reference: ironcore/layers/layernorm/fused_layer_norm.py)."""

from ironcore_b200.layers.norm import Norm


class LayerNorm(Norm):
    def __init__(self, config):
        m = config.model
        super().__init__(m.d_model, m.ln_eps, rms=False, bias=not m.no_bias,
                         weight_offset=float(getattr(m, "norm_weight_offset", 0.0) or 0.0))
        self.config = config
