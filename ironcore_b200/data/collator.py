"""Batch construction.

pretrain: stack windows of ``seq_len + 1`` tokens -> ``input_ids = t[:, :-1]``, ``labels = t[:, 1:]``.
sft     : First-Fit-Decreasing packing of variable-length conversations into rows of ``max_seq_len``;
          labels are ``-100`` on masked (system / user) ranges, padding and the first token of every
          packed sample; per-sample ``position_ids`` restart at 0 and ``cu_seqlens`` holds the sample
          boundaries of the flat token stream, which the attention kernel uses as document masks.
dpo     : a ``chosen_`` and a ``rejected_`` SFT batch.
(Behavioural reference: ironcore/dataloader/collator.py:17-255.)"""

from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

IGNORE_INDEX = -100


def first_fit_decreasing(lengths: List[int], capacity: int) -> List[List[int]]:
    """Indices of the samples in each bin; samples longer than the capacity are truncated to it."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[List[int]] = []
    space: List[int] = []
    for i in order:
        n = min(lengths[i], capacity)
        for b in range(len(bins)):
            if space[b] >= n:
                bins[b].append(i)
                space[b] -= n
                break
        else:
            bins.append([i])
            space.append(capacity - n)
    return bins


class UniversalCollator:
    """``use_flash_attention`` keeps ``cu_seqlens`` in SFT batches (the sample boundaries the attention kernel
    masks by); ``return_full_attention_mask`` adds ``attention_mask`` ``[rows, S, S]`` (bool, block-diagonal over
    the packed samples, padding excluded) for attention paths that take a materialised mask."""

    def __init__(self, mode: str, max_seq_len: int, pad_token_id: int = 0, pack: bool = True,
                 use_flash_attention: bool = True, return_full_attention_mask: bool = False):
        self.mode, self.max_seq_len, self.pad, self.pack = mode, max_seq_len, pad_token_id, pack
        self.pad_token_id = pad_token_id
        self.use_flash_attention = use_flash_attention
        self.return_full_attention_mask = return_full_attention_mask

    def __call__(self, samples: List[Dict]) -> Dict[str, torch.Tensor]:
        if self.mode == "pretrain":
            return self._pretrain(samples)
        if self.mode == "sft":
            return self._sft(samples)
        if self.mode == "dpo":
            # one sample per row, in order: row i of the chosen half pairs with row i of the rejected half
            chosen = self._sft([s["chosen"] for s in samples], pack=False)
            rejected = self._sft([s["rejected"] for s in samples], pack=False)
            out = {f"chosen_{k}": v for k, v in chosen.items()}
            out.update({f"rejected_{k}": v for k, v in rejected.items()})
            return out
        raise ValueError(f"unknown collate mode {self.mode}")

    def _pretrain(self, samples):
        t = torch.from_numpy(np.stack([s["tokens"] for s in samples])).long()
        return {"input_ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous()}

    def _sft(self, samples, pack=None):
        cap = self.max_seq_len + 1
        lengths = [len(s["tokens"]) for s in samples]
        pack = self.pack if pack is None else pack
        bins = first_fit_decreasing(lengths, cap) if pack else [[i] for i in range(len(samples))]
        rows = len(bins)
        tokens = torch.full((rows, cap), self.pad, dtype=torch.long)
        labels_full = torch.full((rows, cap), IGNORE_INDEX, dtype=torch.long)
        pos = torch.zeros((rows, cap), dtype=torch.long)
        boundaries = [0]
        full_mask = torch.zeros((rows, cap, cap), dtype=torch.bool) if self.return_full_attention_mask else None
        for r, members in enumerate(bins):
            col = 0
            for i in members:
                tk = torch.from_numpy(np.asarray(samples[i]["tokens"][:cap - col])).long()
                n = len(tk)
                if n == 0:
                    continue
                tokens[r, col:col + n] = tk
                lab = tk.clone()
                for a, b in samples[i].get("mask_ranges", []):
                    lab[a:min(b, n)] = IGNORE_INDEX
                labels_full[r, col:col + n] = lab
                labels_full[r, col] = IGNORE_INDEX          # never predict a sample's first token from the previous one
                pos[r, col:col + n] = torch.arange(n)
                if full_mask is not None:
                    full_mask[r, col:col + n, col:col + n] = True
                col += n
                boundaries.append(r * self.max_seq_len + min(col, self.max_seq_len))
            if boundaries[-1] != (r + 1) * self.max_seq_len:
                boundaries.append((r + 1) * self.max_seq_len)
        cu = torch.tensor(sorted(set(boundaries)), dtype=torch.int32)
        out = {"input_ids": tokens[:, :-1].contiguous(), "labels": labels_full[:, 1:].contiguous(),
               "position_ids": pos[:, :-1].contiguous(), "loss_mask": (labels_full[:, 1:] != IGNORE_INDEX)}
        if self.use_flash_attention:
            out["cu_seqlens"] = cu
        if full_mask is not None:
            out["attention_mask"] = full_mask[:, :-1, :-1].contiguous()
        return out


def create_collator(mode: str, max_seq_len: int, pad_token_id: int = 0, **kwargs) -> UniversalCollator:
    return UniversalCollator(mode=mode, max_seq_len=max_seq_len, pad_token_id=pad_token_id, **kwargs)
