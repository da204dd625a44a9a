"""Embedding layer built from the configuration (reference: ironcore/layers/embedding.py:9-50)."""

import math

import torch

from ironcore_b200.layers import embedding as _emb


def _vocab_sizes(config):
    """(padded, real) vocabulary size: the registered tokenizer's when there is one, else the configuration's."""
    from ironcore_b200 import global_vars
    from ironcore_b200.parallel import mesh

    tok = global_vars.get_tokenizer()
    m = config.model
    vocab = getattr(tok, "vocab_size", None) or m.vocab_size or config.data.vocab_size
    padded = getattr(tok, "padded_vocab_size", None) or m.padded_vocab_size
    if not padded:
        unit = config.trainer.vocab_padding_unit * mesh.get_tensor_model_parallel_world_size()
        padded = math.ceil(int(vocab) / unit) * unit
    return int(padded), int(vocab)


class LanguageModelEmbedding(_emb.LanguageModelEmbedding):
    """``forward(input_ids [b, s], position_ids [b, s] or None) -> [b, s, d_model]``."""

    def __init__(self, config):
        m = config.model
        padded, vocab = _vocab_sizes(config)
        self.add_position_embedding = m.positional_embedding.type.lower() == "absolute"
        super().__init__(padded, vocab, m.d_model, max(m.max_seq_len, 1), self.add_position_embedding, m.dropout_embd,
                         getattr(m, "embed_scale", None))
        self.config = config

    def forward(self, input_ids: torch.Tensor, position_ids=None) -> torch.Tensor:   # pylint: disable=arguments-differ
        out = super().forward(input_ids, position_ids)
        return out.reshape(*input_ids.shape, -1)
