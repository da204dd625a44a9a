"""Dummy model (reference: ironcore/models/dummy.py:18-65): a stack of fc1 -> ReLU -> fc2 blocks for plumbing tests."""

from ironcore_b200.models import dummy as _d


class DummyModel(_d.DummyModel):
    """``forward(hidden_states, attention_mask, rotary_pos_emb) -> hidden_states``; the two extra arguments are
    accepted and unused, as in the reference."""

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, **kw):   # pylint: disable=arguments-differ
        if isinstance(attention_mask, int) or kw:   # token-major call of the inner stack: (x, seq_len, ...)
            return super().forward(hidden_states, attention_mask, rotary_pos_emb, **kw)
        return super().forward(hidden_states)[0]
