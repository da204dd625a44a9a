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

    @staticmethod
    def apply_rotary_pos_emb(x, sin_emb, cos_emb):
        """Rotate adjacent pairs ``(x[..., 2i], x[..., 2i+1])`` by the angles whose sines / cosines are given
        (broadcastable to ``x[..., ::2]``)."""
        import torch

        x1, x2 = x[..., ::2], x[..., 1::2]
        return torch.stack([x1 * cos_emb - x2 * sin_emb, x1 * sin_emb + x2 * cos_emb], dim=-1).flatten(-2)
