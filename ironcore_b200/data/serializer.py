"""Tokenise datasets into the binary training format.

Per dataset the output directory holds
  ``data.bin``      flat token ids (uint16 when every id < 65535, else uint32)
  ``data.idx.npy``  structured array, one record per sample:
                    (offset u64, length u32, type U20, group_id i64, mask_ranges U500)
                    ``mask_ranges`` is a JSON list of [start, end) token ranges excluded from the loss, or
                    ``@first:count`` pointing at rows of ``data.ranges.npy`` when the JSON does not fit
  ``data.ranges.npy`` int64 [n, 2] side table of the mask ranges that overflow the 500-character field
                    (long conversations); ranges are never truncated
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
BIN_NAME, IDX_NAME, RANGES_NAME = "data.bin", "data.idx.npy", "data.ranges.npy"
MASK_FIELD_CHARS = 500


def encode_mask_ranges(masks: List[List[int]], side_table: List[List[int]]) -> str:
    """Index-record form of ``masks``: the JSON text when it fits the fixed-width field, else a
    reference ``@first:count`` to rows appended to ``side_table``."""
    text = json.dumps(masks, separators=(",", ":"))
    if len(text) <= MASK_FIELD_CHARS:
        return text
    first = len(side_table)
    side_table.extend([int(a), int(b)] for a, b in masks)
    return f"@{first}:{len(masks)}"


def decode_mask_ranges(field: str, side_table) -> List[List[int]]:
    field = str(field)
    if not field:
        return []
    if field.startswith("@"):
        first, count = (int(x) for x in field[1:].split(":"))
        if side_table is None or first + count > len(side_table):
            raise ValueError(f"mask range reference {field} points outside {RANGES_NAME}")
        return [[int(a), int(b)] for a, b in side_table[first:first + count]]
    return json.loads(field)


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
    def __init__(self, config: UniversalDataConfig, tokenizer, verbose: bool = False):
        self.config = config
        self.tok = tokenizer
        self.verbose = verbose

    # ---- per-task tokenisation: yields (tokens, type, group_id, mask_ranges) ----
    def _pretrain(self, ds, rows):
        eos = self.tok.eos_token_id
        for i, row in enumerate(rows):
            text = row.get(ds.text_column)
            if not text:
                continue
            yield list(self.tok.encode(text)) + [eos], "pretrain", i, []

    def _template_tokens(self, messages, template: Optional[str]):
        """Tokens through the tokenizer's own chat template (or ``template``), or None when the tokenizer
        has none. The mask covers every non-assistant turn: turn ``i`` spans the tokens that rendering
        ``messages[:i + 1]`` adds to rendering ``messages[:i]``.
        (Behavioural reference: ironcore/preprocessing/serializer.py:363-410, which measures each turn
        by rendering it alone.)"""
        backend = getattr(self.tok, "backend", None) or self.tok
        fn = getattr(backend, "apply_chat_template", None)
        if fn is None or not (template or getattr(backend, "chat_template", None)):
            return None
        kw = dict(tokenize=True, add_generation_prompt=False)
        if template:
            kw["chat_template"] = template

        def render(msgs):
            out = fn(msgs, **kw)
            if isinstance(out, dict):
                out = out["input_ids"]
            return [int(t) for t in out]

        tokens = render(messages)
        masks: List[List[int]] = []
        prev = 0
        for i, m in enumerate(messages):
            try:
                upto = render(messages[:i + 1])
                end = len(upto) if tokens[:len(upto)] == upto else None
            except Exception:       # templates that reject a conversation ending on this role
                end = None
            if end is None:
                end = min(len(tokens), prev + len(render([m])))
            if i == len(messages) - 1:
                end = len(tokens)
            if m.get("role", "user") != "assistant" and end > prev:
                masks.append([prev, end])
            prev = max(prev, end)
        return tokens, masks

    def _chat_tokens(self, messages, template: Optional[str] = None) -> Tuple[List[int], List[List[int]]]:
        """Chat tokens and masked ranges. With a chat template (the dataset's ``chat_template`` or the
        tokenizer's own) the template decides the text; otherwise turns are concatenated as
        ``<|role|>\\n content \\n``. Every non-assistant turn is masked."""
        rendered = self._template_tokens(messages, template)
        if rendered is not None:
            tokens, masks = rendered
            return tokens, self._merge(masks)
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
        return tokens, self._merge(masks)

    @staticmethod
    def _merge(masks: List[List[int]]) -> List[List[int]]:
        merged: List[List[int]] = []
        for a, b in masks:
            if merged and merged[-1][1] >= a:
                merged[-1][1] = max(merged[-1][1], b)
            else:
                merged.append([a, b])
        return merged

    def _sft(self, ds, rows):
        for i, row in enumerate(rows):
            msgs = row.get(ds.messages_column)
            if not msgs:
                continue
            tokens, masks = self._chat_tokens(msgs, ds.chat_template)
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
                tokens, masks = self._chat_tokens(conv, ds.chat_template)
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
        side_ranges: List[List[int]] = []
        offset = 0
        tmp = out / (BIN_NAME + ".tmp")
        with open(tmp, "wb") as fh:
            for tokens, kind, gid, masks in gen:
                arr = np.asarray(tokens, dtype=dtype)
                fh.write(arr.tobytes())
                records.append((offset, len(arr), kind, gid, encode_mask_ranges(masks, side_ranges)))
                offset += len(arr)
        tmp.replace(out / BIN_NAME)
        idx = np.array(records, dtype=IDX_DTYPE) if records else np.zeros(0, dtype=IDX_DTYPE)
        np.save(out / IDX_NAME, idx)
        if side_ranges:
            np.save(out / RANGES_NAME, np.asarray(side_ranges, dtype=np.int64).reshape(-1, 2))
        elif (out / RANGES_NAME).exists():
            (out / RANGES_NAME).unlink()
        (out / "meta.json").write_text(json.dumps({"dtype": np.dtype(dtype).name, "num_tokens": int(offset),
                                                   "num_samples": len(records), "task_type": ds.task_type,
                                                   "name": ds.name}))
        return out

    def serialize_dataset(self, dataset_config: DatasetConfig, force: bool = False) -> Path:
        """One dataset -> its ``data.bin`` / ``data.idx.npy`` directory (skipped when already there)."""
        if self.verbose:
            print(f"[{dataset_config.name}] task {dataset_config.task_type}, source {dataset_config.source}")
        out = self.serialize(dataset_config, force)
        if self.verbose:
            print(f"[{dataset_config.name}] -> {out}")
        return out

    def serialize_all(self, force: bool = False) -> List[Path]:
        return [self.serialize_dataset(ds, force) for ds in self.config.all_datasets()]
