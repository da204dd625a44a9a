"""Vocabulary-parallel cross entropy (reference: ironcore/parallel/tensor_parallel/cross_entropy.py:22-110)."""

from ironcore_b200.parallel import tensor_parallel as _tp


def vocab_parallel_cross_entropy(vocab_parallel_logits, labels, padding_start_idx=None):
    """Per-token loss of vocabulary-sharded logits; ``padding_start_idx`` is the first padded (unused) vocabulary
    id, whose columns stay out of the softmax."""
    return _tp.vocab_parallel_cross_entropy(vocab_parallel_logits, labels, vocab_size=padding_start_idx)
