"""Tokenizer construction (reference: ironcore/tokenizer/tokenizer.py:26-220)."""

from ironcore_b200.tokenizer import Tokenizer, build_tokenizer  # noqa: F401
