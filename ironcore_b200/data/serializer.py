"""Tokenise datasets into the binary training format.

Per dataset the output directory holds
  ``data.bin``      flat token ids (uint16 when every id < 65535, else uint32)
  ``data.idx.npy``  structured array, one record per sample:
                    (offset u64, length u32, type U20, group_id i64, mask_ranges U500)
                    ``mask_ranges`` is a JSON list of [start, end) token ranges excluded from the loss
pretrain: one record per document (document + EOS); sft: chat-formatted tokens with the
system / user turns masked; dpo: a chosen and a rejected record sharing ``group_id``.
Sources: a local ``.jsonl`` / ``.json`` / ``.txt`` file or directory, or a HuggingFace dataset name
when the ``datasets`` package can serve it from its local cache.
(Behavioural reference: ironcore/preprocessing/serializer.py:17-437.)"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import numpy as np

from .data_config import DatasetConfig, UniversalDataConfig

IDX_DTYPE = np.dtype([("offset", "<u8"), ("length", "<u4"), ("type", "<U20"), ("group_id", "<i8"),
                      ("mask_ranges", "<U500")])
BIN_NAME, IDX_NAME = "data.bin", "data.idx.npy"


def _iter_local(path: Path) -> Iterator[Dict]:
    files = sorted(p for p in path.rglob("*") if p.suffix in (".jsonl", ".json", ".txt")) if path.is_dir() else [path]
    for f in files:
        if f.suffix == ".jsonl":
            with open(f, encoding="utf-8") as fh:
                for line in fh:
                    line = line.strip()
                    if line:
                        yield json.loads(line)
        elif f.suffix == ".json":
            doc = json.loads(f.read_text(encoding="utf-8"))
            for row in (doc if isinstance(doc, list) else doc.get("data", [doc])):
                yield row
        else:
            for block in f.read_text(encoding="utf-8").split("\n\n"):
                if block.strip():
                    yield {"text": block.strip()}


def load_rows(ds: DatasetConfig, cache_dir: Optional[Path] = None) -> Iterable[Dict]:
    src = Path(ds.source)
    if src.exists():
        rows = _iter_local(src)
    else:
        try:
            from datasets import load_dataset
        except Exception as exc:
            raise FileNotFoundError(f"dataset source {ds.source} is not a local path and the `datasets` package "
                                    f"is unavailable") from exc
        rows = load_dataset(ds.source, ds.subset, split=ds.split, cache_dir=str(cache_dir) if cache_dir else None)
    if ds.max_samples is not None:
        def limited(it, n):
            for i, r in enumerate(it):
                if i >= n:
                    return
                yield r
        rows = limited(rows, ds.max_samples)
    return rows


class DataSerializer:
    def __init__(self, config: UniversalDataConfig, tokenizer):
        self.config = config
        self.tok = tokenizer

    # ---- per-task tokenisation: yields (tokens, type, group_id, mask_ranges) ----
    def _pretrain(self, ds, rows):
        eos = self.tok.eos_token_id
        for i, row in enumerate(rows):
            text = row.get(ds.text_column)
            if not text:
                continue
            yield list(self.tok.encode(text)) + [eos], "pretrain", i, []

    def _chat_tokens(self, messages) -> Tuple[List[int], List[List[int]]]:
        """Concatenate turns as ``<|role|>\\n content \\n``; every non-assistant turn is masked."""
        tokens: List[int] = []
        masks: List[List[int]] = []
        for m in messages:
            role, content = m.get("role", "user"), m.get("content", "")
            header = self.tok.encode(f"<|{role}|>\n")
            body = self.tok.encode(content + "\n")
            start = len(tokens)
            tokens.extend(header)
            if role == "assistant":
                masks.append([start, len(tokens)])      # the header itself is not a prediction target
                tokens.extend(body)
                tokens.append(self.tok.eos_token_id)
            else:
                tokens.extend(body)
                masks.append([start, len(tokens)])
        merged: List[List[int]] = []
        for a, b in masks:
            if merged and merged[-1][1] >= a:
                merged[-1][1] = max(merged[-1][1], b)
            else:
                merged.append([a, b])
        return tokens, merged

    def _sft(self, ds, rows):
        for i, row in enumerate(rows):
            msgs = row.get(ds.messages_column)
            if not msgs:
                continue
            tokens, masks = self._chat_tokens(msgs)
            yield tokens, "sft", i, masks

    def _dpo(self, ds, rows):
        for i, row in enumerate(rows):
            chosen, rejected = row.get(ds.chosen_column), row.get(ds.rejected_column)
            if not chosen or not rejected:
                continue
            for kind, conv in (("dpo_chosen", chosen), ("dpo_rejected", rejected)):
                if isinstance(conv, str):
                    conv = [{"role": "assistant", "content": conv}]
                    if row.get("prompt"):
                        conv = [{"role": "user", "content": row["prompt"]}] + conv
                tokens, masks = self._chat_tokens(conv)
                yield tokens, kind, i, masks

    # ---- writing ----
    def is_serialized(self, ds: DatasetConfig) -> bool:
        out = Path(ds.output_path)
        return (out / BIN_NAME).exists() and (out / IDX_NAME).exists()

    def serialize(self, ds: DatasetConfig, force: bool = False) -> Path:
        out = Path(ds.output_path)
        if self.is_serialized(ds) and not force:
            return out
        out.mkdir(parents=True, exist_ok=True)
        rows = load_rows(ds, self.config.cache_dir)
        gen = {"pretrain": self._pretrain, "sft": self._sft, "dpo": self._dpo}[ds.task_type](ds, rows)
        vocab = getattr(self.tok, "vocab_size", 1 << 20)
        dtype = np.uint16 if vocab < 65535 else np.uint32
        records = []
        offset = 0
        tmp = out / (BIN_NAME + ".tmp")
        with open(tmp, "wb") as fh:
            for tokens, kind, gid, masks in gen:
                arr = np.asarray(tokens, dtype=dtype)
                fh.write(arr.tobytes())
                mr = json.dumps(masks)
                if len(mr) > 500:
                    mr = json.dumps(masks[: max(1, len(masks) // 2)])[:500]
                records.append((offset, len(arr), kind, gid, mr))
                offset += len(arr)
        tmp.replace(out / BIN_NAME)
        idx = np.array(records, dtype=IDX_DTYPE) if records else np.zeros(0, dtype=IDX_DTYPE)
        np.save(out / IDX_NAME, idx)
        (out / "meta.json").write_text(json.dumps({"dtype": np.dtype(dtype).name, "num_tokens": int(offset),
                                                   "num_samples": len(records), "task_type": ds.task_type,
                                                   "name": ds.name}))
        return out

    def serialize_all(self, force: bool = False) -> List[Path]:
        return [self.serialize(ds, force) for ds in self.config.all_datasets()]
