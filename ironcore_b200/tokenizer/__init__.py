"""Tokenizer abstraction. HuggingFace tokenizers are used when their files are available
locally (no network access is attempted: ``local_files_only``); otherwise a vocab-size-only
stub supplies the ids the model and the data pipeline need.
(Behavioural reference: ironcore/tokenizer/tokenizer.py:26-220.)"""

from __future__ import annotations

import math
import os
from typing import List, Optional

_KNOWN_VOCAB = {"gpt2": 50257, "bbpe": 50257, "tiktoken": 50257, "llama": 32000, "sentencepiece": 32000,
                "qwen": 151936, "t5": 32100}


def pad_vocab_size(vocab_size: int, unit: int, tp_size: int = 1) -> int:
    mult = unit * max(tp_size, 1)
    return int(math.ceil(vocab_size / mult) * mult)


class Tokenizer:
    """Common surface: vocab_size, padded_vocab_size, eos/eod/pad ids, encode/decode."""

    def __init__(self, vocab_size: int, eos_token_id: int, pad_token_id: Optional[int], padding_unit: int = 128,
                 tp_size: int = 1, backend=None, eos_token: str = "<|endoftext|>"):
        self.vocab_size = int(vocab_size)
        self.eos_token_id = int(eos_token_id)
        self.eod_token_id = int(eos_token_id)
        self.pad_token_id = int(pad_token_id if pad_token_id is not None and pad_token_id >= 0 else eos_token_id)
        self.eos_token = eos_token
        self.padded_vocab_size = pad_vocab_size(self.vocab_size, padding_unit, tp_size)
        self.backend = backend

    def encode(self, text: str) -> List[int]:
        if self.backend is not None:
            return list(self.backend.encode(text))
        # deterministic byte-level fallback: bytes map to ids [0, 256)
        return [b % self.vocab_size for b in text.encode("utf-8")]

    def decode(self, ids) -> str:
        if self.backend is not None:
            return self.backend.decode(list(ids))
        return bytes([int(i) % 256 for i in ids]).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, **kw):
        if self.backend is not None and hasattr(self.backend, "apply_chat_template"):
            return self.backend.apply_chat_template(messages, **kw)
        return "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages)

    def __len__(self):
        return self.vocab_size


def _try_hf(name_or_path: str, tokenizer_type: str):
    try:
        os.environ.setdefault("HF_HUB_OFFLINE", "1")
        if tokenizer_type in ("bbpe", "gpt2", "tiktoken"):
            from transformers import GPT2TokenizerFast as Cls
        else:
            from transformers import AutoTokenizer as Cls
        if not name_or_path or str(name_or_path).lower() in ("none", "stub"):
            return None
        tok = Cls.from_pretrained(name_or_path, local_files_only=True)
        # a tokenizer built without its vocabulary files encodes everything to nothing: reject it
        if len(tok.encode("hello world")) == 0 or len(tok) < 256:
            return None
        return tok
    except Exception:
        return None


def build_tokenizer(config) -> Tokenizer:
    m = config.model
    tp = config.trainer.tensor_model_parallel_size
    unit = config.trainer.vocab_padding_unit
    ttype = str(m.tokenizer_type).lower()
    hf = None
    if getattr(config.data, "task_type", "pretrain") != "synthetic":
        hf = _try_hf(m.vocab_name_or_path, ttype)
    special = dict(getattr(config.data, "special_tokens", None) or {})
    if hf is not None:
        for name, value in special.items():      # token strings (eos_token, pad_token, ...) of the backend
            if not name.endswith("_id"):
                setattr(hf, name, value)
        eos = hf.eos_token_id if hf.eos_token_id is not None else len(hf) - 1
        tok = Tokenizer(len(hf), eos, hf.pad_token_id, unit, tp, backend=hf, eos_token=hf.eos_token or "")
        eod = getattr(hf, "eod_token", None)
        if eod is not None:
            tok.eod_token_id = int(hf.convert_tokens_to_ids(eod))
    else:
        vocab = m.vocab_size or _KNOWN_VOCAB.get(ttype) or config.data.vocab_size
        eos = vocab - 1
        pad = config.data.pad_token_id
        tok = Tokenizer(vocab, eos, pad, unit, tp, eos_token=special.get("eos_token", "<|endoftext|>"))
    for name in ("eos_token_id", "eod_token_id", "pad_token_id"):    # explicit ids win on either path
        if special.get(name) is not None:
            setattr(tok, name, int(special[name]))
    if "eos_token_id" in special and "eod_token_id" not in special:
        tok.eod_token_id = tok.eos_token_id
    return tok
