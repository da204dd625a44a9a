"""File-backed iterators for the trainer: dataset YAML -> mixing datasets -> DataLoader -> batches."""

from __future__ import annotations

from typing import Dict

import torch
from torch.utils.data import DataLoader

from .collator import UniversalCollator
from .data_config import UniversalDataConfig
from .dataset import WeightedMixingDataset


def build_file_iterators(config, dp_rank: int, dp_size: int) -> Dict[str, object]:
    dcfg = UniversalDataConfig.from_yaml(config.data.config_path)
    task = str(getattr(config.data, "task_type", "pretrain")).lower()
    seq_len = config.model.max_seq_len
    pad = config.model.pad_token_id if config.model.pad_token_id is not None else 0
    out = {}
    for split in ("train", "eval", "test"):
        sources = {"train": dcfg.datasets, "eval": dcfg.eval_datasets or dcfg.datasets,
                   "test": dcfg.test_datasets or dcfg.datasets}[split]
        enabled = split == "train" or (split == "eval" and config.trainer.do_eval) or \
            (split == "test" and config.trainer.do_test)
        sources = [s for s in sources if s.task_type == task]
        if not enabled or not sources:
            out[split] = None
            continue
        ds = WeightedMixingDataset.from_data_config(dcfg, task, 1337, split, dp_rank, dp_size,
                                                    epochs=None if split == "train" else 1, seq_len=seq_len)
        bs = {"train": config.trainer.micro_batch_size,
              "eval": config.trainer.eval_batch_size or config.trainer.micro_batch_size,
              "test": config.trainer.test_batch_size or config.trainer.micro_batch_size}[split]
        loader = DataLoader(ds, batch_size=bs, collate_fn=UniversalCollator(task, seq_len, pad), num_workers=0,
                            pin_memory=torch.cuda.is_available(), drop_last=(split == "train"))
        out[split] = _BatchIterator(loader, ds, bs)
    return out


class _BatchIterator:
    """Iterator over a loader's batches that can pass over its first batches without reading their tokens."""

    def __init__(self, loader, dataset, batch_size: int):
        self.loader, self.dataset, self.batch_size = loader, dataset, batch_size
        self._it = None

    def __iter__(self):
        return self

    def __next__(self):
        if self._it is None:
            self._it = iter(self.loader)
        return next(self._it)

    def skip_batches(self, n: int) -> None:
        """Advance the stream by ``n`` batches. Before the first batch was drawn this only moves the dataset's
        starting point (fixed-size samples per batch: pretrain windows, one pair or conversation per sample);
        afterwards the batches are drawn and dropped."""
        if self._it is None:
            self.dataset.start_sample += int(n) * self.batch_size
            return
        for _ in range(int(n)):
            next(self)
