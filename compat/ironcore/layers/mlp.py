"""Feed-forward block built from the configuration (reference: ironcore/layers/mlp.py:19-54)."""

import torch

from ironcore_b200.layers import mlp as _mlp


class MLP(_mlp.MLP):
    """``forward(x [..., d_model]) -> [..., d_model]``; gated activations double the up projection, whose halves
    are sharded separately under tensor parallelism."""

    def __init__(self, config):
        m = config.model
        super().__init__(m.d_model, m.d_ffn, m.activation_type, bias=not m.no_bias, dropout=m.dropout_mlp)
        self.config = m
        self.tensor_model_parallel_size = config.trainer.tensor_model_parallel_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # pylint: disable=arguments-differ
        lead = x.shape[:-1]
        return super().forward(x.reshape(-1, x.shape[-1])).reshape(*lead, -1)
