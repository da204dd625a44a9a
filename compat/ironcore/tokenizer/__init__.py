"""Tokenizers (reference: ironcore/tokenizer/__init__.py)."""

from .tokenizer import BbpeTokenizer, SentencePieceTokenizer, Tokenizer, build_tokenizer  # noqa: F401
