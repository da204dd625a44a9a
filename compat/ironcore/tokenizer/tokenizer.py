"""Tokenizer wrappers with the reference's constructors (reference: ironcore/tokenizer/tokenizer.py:26-220):
``Tokenizer(tokenizer, vocab_name_or_path, vocab_padding_unit, special_tokens_config)`` wraps a loaded
HuggingFace-style tokenizer object; ``BbpeTokenizer`` / ``SentencePieceTokenizer`` load one from local files (no
network access is attempted)."""

from __future__ import annotations

from typing import Dict, Optional

from ironcore_b200 import tokenizer as _tok
from ironcore_b200.tokenizer import build_tokenizer, pad_vocab_size  # noqa: F401


class Tokenizer(_tok.Tokenizer):
    def __init__(self, tokenizer, vocab_name_or_path=None, vocab_padding_unit: int = 128,
                 special_tokens_config: Optional[Dict[str, str]] = None):
        for name, value in (special_tokens_config or {}).items():
            setattr(tokenizer, name, value)
        eos_token = (getattr(tokenizer, "eot_token", None) or getattr(tokenizer, "eod_token", None)
                     or getattr(tokenizer, "eos_token", None))
        if eos_token is None:
            raise ValueError("eos_token not found in the tokenizer: check special_tokens_config or the tokenizer files")
        if getattr(tokenizer, "pad_token", None) is None:
            tokenizer.pad_token = tokenizer.eos_token
        vocab = getattr(tokenizer, "vocab_size", None) or getattr(tokenizer, "n_vocab", None)
        if vocab is None:
            raise ValueError("the tokenizer has neither vocab_size nor n_vocab")
        try:
            vocab = max(int(vocab), len(tokenizer))     # added / special tokens sit above the base vocabulary
        except TypeError:
            vocab = int(vocab)
        super().__init__(vocab, tokenizer.eos_token_id, getattr(tokenizer, "pad_token_id", None), vocab_padding_unit,
                         1, backend=tokenizer, eos_token=eos_token)
        self._tokenizer = tokenizer
        self.vocab_name_or_path = vocab_name_or_path
        eod = getattr(tokenizer, "eod_token_id", None)
        if eod is not None:
            self.eod_token_id = int(eod)

    @property
    def pad_token(self):
        return self._tokenizer.pad_token

    def __call__(self, *args, **kwargs):
        """The wrapped tokenizer's own call (a batch encoding with ``input_ids``), as in the reference."""
        return self._tokenizer(*args, **kwargs)

    def decode(self, token_ids) -> str:   # pylint: disable=arguments-renamed
        return super().decode(token_ids) if len(token_ids) else ""

    def __str__(self):
        return (f"Tokenizer type: {type(self).__name__}\nVocab path: {self.vocab_name_or_path}\n"
                f"Vocab size: {self.vocab_size}\nPadded vocab size: {self.padded_vocab_size}\n"
                f"EOS token: {self.eos_token}\n")


def _load(name_or_path, kind: str):
    backend = _tok._try_hf(str(name_or_path), kind)   # pylint: disable=protected-access
    if backend is None:
        raise FileNotFoundError(f"no usable {kind} tokenizer files at {name_or_path!r} (only local files are read)")
    return backend


class BbpeTokenizer(Tokenizer):
    def __init__(self, vocab_name_or_path, merge_file_path=None, vocab_padding_unit: int = 128,
                 special_tokens_config: Optional[Dict[str, str]] = None):
        if merge_file_path:
            from transformers import GPT2TokenizerFast

            backend = GPT2TokenizerFast(vocab_file=str(vocab_name_or_path), merges_file=str(merge_file_path))
        else:
            backend = _load(vocab_name_or_path, "gpt2")
        super().__init__(backend, vocab_name_or_path, vocab_padding_unit, special_tokens_config)


class SentencePieceTokenizer(Tokenizer):
    def __init__(self, vocab_name_or_path, vocab_padding_unit: int = 128,
                 special_tokens_config: Optional[Dict[str, str]] = None):
        super().__init__(_load(vocab_name_or_path, "sentencepiece"), vocab_name_or_path, vocab_padding_unit,
                         special_tokens_config)
