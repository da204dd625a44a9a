"""Rotary positional embedding with the reference's constructor
(reference: ironcore/layers/positional_embedding/rotary.py:15-83)."""

from ironcore_b200.layers import positional as _pos


class RotaryPositionalEmbedding(_pos.RotaryPositionalEmbedding):
    """``forward(x [b, s, heads, head_dim])`` rotates adjacent pairs by the angle of the *sequence* position
    (``offset`` + index, times ``scale``). ``max_seq_len`` is accepted for the signature; no table is cached."""

    def __init__(self, head_dim: int, max_seq_len: int = 4096, base: float = 10000, scale: float = 1.0, offset: int = 0):
        super().__init__(head_dim, base=float(base), scaling_factor=float(scale), offset=int(offset), interleaved=True)
        self.max_seq_len = max_seq_len
        self.rope_base, self.scale = base, scale
