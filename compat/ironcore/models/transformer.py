"""Transformer stack with the reference's layer-level call convention
(reference: ironcore/models/transformer.py:23-162): ``TransformerLayer(config)`` and ``TransformerModel(config)``
take ``hidden_states [b, s, d]``, an attention mask (positions equal to 0 are masked out; not read when
``trainer.use_flash_attn`` selects the causal flash kernel) and an optional rotary embedding module."""

from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint

from ironcore_b200.layers.module import init_parameters
from ironcore_b200.models import transformer as _t


class _ProjectionView:
    """A logical projection inside the fused q|k|v parameter: ``weight`` ``[in, out_local]`` and ``bias`` are views
    of the fused tensors, so reading or writing them in place reads or writes the layer's parameters."""

    def __init__(self, fused, lo: int, hi: int):
        self._fused, self._lo, self._hi = fused, lo, hi

    @property
    def weight(self):
        return self._fused.weight[:, self._lo:self._hi]

    @property
    def bias(self):
        return None if self._fused.bias is None else self._fused.bias[self._lo:self._hi]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = x.reshape(-1, x.shape[-1]) @ self.weight
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*x.shape[:-1], -1)


class TransformerLayer(_t.TransformerLayer):
    def __init__(self, config, layer_idx: int = 0, dtype=None, device=None):
        super().__init__(config, layer_idx, dtype, device)
        self.config, self.model_config, self.init_config = config, config.model, config.init
        self.head_dimension = self.head_dim
        self.num_local_attention_heads, self.num_local_attention_groups = self.heads_local, self.kv_heads_local
        self._flash = bool(config.trainer.use_flash_attn)
        # the reference's standard attention masks only what the mask names; its flash path is always causal
        self.attention.causal = self._flash

    # -- the reference's attribute names ---------------------------------------------------------------
    @property
    def self_attention(self):
        return self.attention

    @property
    def linear_q(self):
        return _ProjectionView(self.linear_qkv, 0, self.heads_local * self.head_dim)

    @property
    def linear_kv(self):
        q = self.heads_local * self.head_dim
        return _ProjectionView(self.linear_qkv, q, q + 2 * self.kv_heads_local * self.head_dim)

    def init_weights(self):
        init_parameters(self, self.config)

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None):   # pylint: disable=arguments-differ
        if hidden_states.dim() == 2:   # token-major call of the inner stack: (x, seq_len, pos_ids, cu_seqlens, ...)
            return super().forward(hidden_states, attention_mask, rotary_pos_emb)
        b, s, d = hidden_states.shape
        mask = None
        if attention_mask is not None and not self._flash:
            mask = attention_mask != 0
        att = self.attention
        own = att._modules.get("rotary", att.__dict__.get("rotary"))   # pylint: disable=protected-access
        att.__dict__.pop("rotary", None)
        att._modules["rotary"] = rotary_pos_emb if rotary_pos_emb is not None else None   # pylint: disable=protected-access
        try:
            out, _aux, _ = super().forward(hidden_states.reshape(b * s, d), s, attn_mask=mask)
        finally:
            att._modules["rotary"] = own   # pylint: disable=protected-access
        return out.reshape(b, s, d)

    custom_forward = forward


class TransformerModel(_t.TransformerModel):
    def __init__(self, config, dtype=None, device=None):
        super().__init__(config, dtype, device)
        self.layers = torch.nn.ModuleList([TransformerLayer(config, i, dtype, device)
                                           for i in range(config.model.num_layers)])

    def init_weights(self):
        init_parameters(self, self.config)

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None):   # pylint: disable=arguments-differ
        if hidden_states.dim() == 2:
            return super().forward(hidden_states, attention_mask, rotary_pos_emb)
        for layer in self.layers:
            if self.recompute and self.training:
                hidden_states = checkpoint(layer.custom_forward, hidden_states, attention_mask, rotary_pos_emb,
                                           use_reentrant=self.use_reentrant)
            else:
                hidden_states = layer(hidden_states, attention_mask, rotary_pos_emb)
        return hidden_states
