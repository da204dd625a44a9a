"""HellaSwag: four candidate endings per context; the prediction is the ending with the lowest mean
per-token cross entropy; score = accuracy in percent. Examples come from the HuggingFace dataset
cache, a local JSONL file (``HELLASWAG_PATH`` or ``<cache_dir>/hellaswag.jsonl``), or are passed in.
(Behavioural reference: ironcore/eval/tasks/hellaswag.py:24-172.)"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, Iterable

import torch

from .base_task import Task


class HellaSwag(Task):
    name = "hellaswag"
    metric = "accuracy"

    def load_examples(self) -> Iterable[dict]:
        local = os.environ.get("HELLASWAG_PATH") or (Path(self.cache_dir) / "hellaswag.jsonl" if self.cache_dir else None)
        if local and Path(local).exists():
            with open(local) as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)
            return
        try:
            from datasets import load_dataset

            for row in load_dataset("hellaswag", split="validation", cache_dir=str(self.cache_dir) if self.cache_dir else None):
                yield row
        except Exception as exc:
            raise FileNotFoundError("HellaSwag examples are unavailable offline; set HELLASWAG_PATH to a JSONL file "
                                    "with fields ctx, endings, label") from exc

    @torch.no_grad()
    def score_example(self, model, ctx: str, endings) -> torch.Tensor:
        """Mean cross entropy of each ending given the context, one forward pass over the 4 rows."""
        dev = next(model.parameters()).device
        ctx_ids = self.tokenizer.encode(ctx)
        rows, spans = [], []
        for e in endings:
            end_ids = self.tokenizer.encode(" " + e)
            rows.append(ctx_ids + end_ids)
            spans.append((len(ctx_ids), len(ctx_ids) + len(end_ids)))
        width = max(len(r) for r in rows)
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        ids = torch.full((len(rows), width), pad, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, :len(r)] = torch.tensor(r)
        ids = ids.to(dev)
        tgt = ids[:, 1:]
        scorer = getattr(getattr(model, "module", model), "token_logprobs", None)
        if scorer is not None:
            # vocab-parallel cross entropy: correct under tensor parallelism (every rank holds a vocabulary
            # shard of the logits and the three per-token scalars are exchanged), and no [rows, vocab] softmax
            tok_lp = scorer(ids[:, :-1], tgt).float()
        else:
            logits = model(ids[:, :-1]).float()
            vocab = getattr(model, "vocab_size", logits.shape[-1])
            logp = torch.log_softmax(logits[..., :vocab], dim=-1)
            tok_lp = logp.gather(-1, tgt.unsqueeze(-1)).squeeze(-1)
        out = []
        for i, (a, b) in enumerate(spans):
            out.append(-tok_lp[i, a - 1:b - 1].mean())
        return torch.stack(out)

    def process(self, model) -> Dict[str, float]:
        correct = total = 0
        for ex in self.examples():
            losses = self.score_example(model, ex["ctx"], ex["endings"])
            correct += int(int(losses.argmin()) == int(ex["label"]))
            total += 1
        return {"metric": self.metric, "score": 100.0 * correct / max(total, 1)}
