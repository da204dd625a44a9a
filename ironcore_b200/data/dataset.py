"""Memory-mapped datasets over the binary format and weighted mixing of several sources.

pretrain: fixed windows of ``seq_len + 1`` tokens starting every ``seq_len`` tokens (wrapping at the
end); an epoch draws ``round(N * ratio_i)`` windows from source ``i`` (N = windows of all sources; a
source smaller than its share is revisited, a larger one is subsampled without replacement), in a
seeded shuffle sharded ``index % dp_size == dp_rank``; sft / dpo: samples
drawn by weighted sampling without replacement, then rank-sharded. Train / eval / test splits are
contiguous token (pretrain) or sample (sft, dpo) ranges given by the split ratios.
(Behavioural reference: ironcore/dataloader/universal_dataset.py:20-390.)"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterator, List, Optional

import numpy as np
from torch.utils.data import IterableDataset

from .serializer import BIN_NAME, IDX_NAME, RANGES_NAME, decode_mask_ranges


class BinaryDataset:
    def __init__(self, directory):
        d = Path(directory)
        if not (d / BIN_NAME).exists() or not (d / IDX_NAME).exists():
            raise FileNotFoundError(f"{d} does not contain {BIN_NAME} / {IDX_NAME}; run `ironcore preprocess`")
        self.index = np.load(d / IDX_NAME, allow_pickle=False)
        meta = d / "meta.json"
        if meta.exists():
            dtype = np.dtype(json.loads(meta.read_text())["dtype"])
        else:
            nbytes = (d / BIN_NAME).stat().st_size
            total = int(self.index["offset"][-1] + self.index["length"][-1]) if len(self.index) else 0
            dtype = np.dtype(np.uint16) if total and nbytes // total == 2 else np.dtype(np.uint32)
        self.tokens = np.memmap(d / BIN_NAME, dtype=dtype, mode="r")
        self.ranges = np.load(d / RANGES_NAME, allow_pickle=False) if (d / RANGES_NAME).exists() else None
        self.directory = d

    @property
    def num_tokens(self) -> int:
        return int(self.tokens.shape[0])

    def __len__(self) -> int:
        return len(self.index)

    def sample(self, i: int) -> Dict:
        rec = self.index[i]
        o, n = int(rec["offset"]), int(rec["length"])
        return {"tokens": np.asarray(self.tokens[o:o + n], dtype=np.int64), "type": str(rec["type"]),
                "group_id": int(rec["group_id"]), "mask_ranges": decode_mask_ranges(rec["mask_ranges"], self.ranges)}

    def window(self, start: int, length: int) -> np.ndarray:
        """``length`` tokens from ``start`` (wrapping around the end of the corpus)."""
        total = self.num_tokens
        start %= max(total, 1)
        if start + length <= total:
            return np.asarray(self.tokens[start:start + length], dtype=np.int64)
        head = np.asarray(self.tokens[start:], dtype=np.int64)
        reps = [head]
        need = length - len(head)
        while need > 0:
            part = np.asarray(self.tokens[:min(need, total)], dtype=np.int64)
            reps.append(part)
            need -= len(part)
        return np.concatenate(reps)


def _split_range(n: int, splits: List[float], split: str):
    idx = {"train": 0, "eval": 1, "test": 2}[split]
    bounds = np.cumsum([0.0] + list(splits))
    lo, hi = int(round(bounds[idx] * n)), int(round(bounds[idx + 1] * n))
    return lo, hi


class WeightedMixingDataset(IterableDataset):
    def __init__(self, directories: List, ratios: List[float], mode: str, split: str, seq_len: int,
                 splits: List[float], seed: int = 1337, dp_rank: int = 0, dp_size: int = 1, epochs: Optional[int] = None):
        self.sets = [BinaryDataset(d) for d in directories]
        w = np.asarray(ratios, dtype=np.float64)
        self.weights = w / w.sum()
        self.mode, self.split, self.seq_len, self.splits = mode, split, seq_len, splits
        self.seed, self.dp_rank, self.dp_size = seed, dp_rank, dp_size
        self.epochs = epochs
        self.cursor = 0          # samples yielded so far on this rank (saved in checkpoints)
        self.start_sample = 0    # samples of this rank's stream to pass over before the first one is read (resume)

    @staticmethod
    def sources_of(data_config, mode: str, split: str) -> Dict:
        """Directories, ratios and split ratios of one split of a dataset YAML (``UniversalDataConfig``): the
        split's own dataset list when it has one (used whole), else the split's share of the training datasets;
        only datasets of task type ``mode`` take part."""
        own = {"train": data_config.datasets, "eval": data_config.eval_datasets, "test": data_config.test_datasets}
        if split not in own:
            raise ValueError(f"Invalid split: {split}")
        separate = split != "train" and bool(own[split])
        sources = [d for d in (own[split] if separate or split == "train" else data_config.datasets)
                   if d.task_type == mode]
        if not sources:
            raise ValueError(f"no {mode} dataset for split {split}")
        return dict(directories=[d.output_path for d in sources], ratios=[d.ratio for d in sources], mode=mode,
                    split="train" if separate else split,
                    splits=[1.0, 0.0, 0.0] if separate else list(data_config.splits))

    @classmethod
    def from_data_config(cls, data_config, mode: str = "pretrain", seed: int = 1337, split: str = "train",
                         dp_rank: int = 0, dp_size: int = 1, epochs: Optional[int] = None, seq_len: Optional[int] = None):
        return cls(seq_len=seq_len or data_config.max_seq_len, seed=seed, dp_rank=dp_rank, dp_size=dp_size,
                   epochs=epochs, **cls.sources_of(data_config, mode, split))

    def _pretrain_positions(self):
        items = []
        for si, ds in enumerate(self.sets):
            lo, hi = _split_range(ds.num_tokens, self.splits, self.split)
            for start in range(lo, max(lo, hi - 1), self.seq_len):
                items.append((si, start))
        return items

    def _weighted_pretrain_order(self, items, rng) -> np.ndarray:
        """Indices into ``items`` for one epoch: every source contributes its ratio's share of the epoch."""
        src = np.asarray([si for si, _ in items])
        total = len(items)
        if len(self.sets) == 1:
            return rng.permutation(total)
        picks = []
        for si in range(len(self.sets)):
            own = np.flatnonzero(src == si)
            want = int(round(total * float(self.weights[si])))
            if len(own) == 0 or want == 0:
                continue
            full, rest = divmod(want, len(own))
            for _ in range(full):
                picks.append(rng.permutation(own))
            if rest:
                picks.append(rng.choice(own, size=rest, replace=False))
        order = np.concatenate(picks) if picks else np.zeros(0, dtype=np.int64)
        return order[rng.permutation(len(order))]

    def _sample_items(self):
        items, probs = [], []
        for si, ds in enumerate(self.sets):
            lo, hi = _split_range(len(ds), self.splits, self.split)
            n = max(hi - lo, 0)
            for i in range(lo, hi):
                items.append((si, i))
                probs.append(self.weights[si] / max(n, 1))
        return items, np.asarray(probs)

    def _passed_over(self) -> bool:
        """Whether the next sample of the stream is one to pass over without reading it (``start_sample``)."""
        if self._to_skip > 0:
            self._to_skip -= 1
            self.cursor += 1
            return True
        return False

    def __iter__(self) -> Iterator[Dict]:
        epoch = 0
        self._to_skip = int(self.start_sample)
        while self.epochs is None or epoch < self.epochs:
            rng = np.random.default_rng(self.seed + epoch)
            if self.mode == "pretrain":
                items = self._pretrain_positions()
                if not items:
                    return
                order = self._weighted_pretrain_order(items, rng)
                for j, k in enumerate(order):
                    if j % self.dp_size != self.dp_rank:
                        continue
                    if self._passed_over():
                        continue
                    si, start = items[k]
                    self.cursor += 1
                    yield {"tokens": self.sets[si].window(start, self.seq_len + 1), "type": "pretrain"}
            else:
                items, probs = self._sample_items()
                if not items:
                    return
                probs = probs / probs.sum()
                order = rng.choice(len(items), size=len(items), replace=False, p=probs)
                if self.mode == "dpo":
                    # keep chosen / rejected of a group together: iterate over group ids
                    seen = set()
                    j = 0
                    for k in order:
                        si, i = items[k]
                        gid = (si, int(self.sets[si].index[i]["group_id"]))
                        if gid in seen:
                            continue
                        seen.add(gid)
                        if j % self.dp_size == self.dp_rank:
                            grp = [x for x in range(len(self.sets[si])) if int(self.sets[si].index[x]["group_id"]) == gid[1]]
                            pair = {str(self.sets[si].index[x]["type"]): self.sets[si].sample(x) for x in grp}
                            if "dpo_chosen" in pair and "dpo_rejected" in pair:
                                if self._passed_over():
                                    j += 1
                                    continue
                                self.cursor += 1
                                yield {"chosen": pair["dpo_chosen"], "rejected": pair["dpo_rejected"], "type": "dpo"}
                        j += 1
                else:
                    for j, k in enumerate(order):
                        if j % self.dp_size != self.dp_rank:
                            continue
                        if self._passed_over():
                            continue
                        si, i = items[k]
                        self.cursor += 1
                        yield self.sets[si].sample(i)
            epoch += 1
