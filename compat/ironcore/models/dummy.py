"""Dummy model (reference: ironcore/models/dummy.py:18-65): a stack of fc1 -> ReLU -> fc2 blocks for plumbing tests."""

from torch import nn

from ironcore_b200.layers.module import BaseModule
from ironcore_b200.models import dummy as _d


class DummyModelLayer(BaseModule):
    """fc1 -> ReLU -> fc2 on the last dimension (``d_model -> d_ffn -> d_model``)."""

    def __init__(self, config):
        super().__init__(config)
        self.model_config, self.init_config = config.model, config.init
        self.hidden_size = config.model.d_ffn
        self.fc1 = nn.Linear(config.model.d_model, config.model.d_ffn)
        self.relu = nn.ReLU()
        self.fc2 = nn.Linear(config.model.d_ffn, config.model.d_model)

    def custom_forward(self, x, attention_mask=None, rotary_pos_emb=None):   # pylint: disable=unused-argument
        return self.fc2(self.relu(self.fc1(x)))

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None):
        return self.custom_forward(hidden_states, attention_mask, rotary_pos_emb)


class DummyModel(_d.DummyModel):
    """``forward(hidden_states, attention_mask, rotary_pos_emb) -> hidden_states``; the two extra arguments are
    accepted and unused, as in the reference."""

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, **kw):   # pylint: disable=arguments-differ
        if isinstance(attention_mask, int) or kw:   # token-major call of the inner stack: (x, seq_len, ...)
            return super().forward(hidden_states, attention_mask, rotary_pos_emb, **kw)
        return super().forward(hidden_states)[0]
