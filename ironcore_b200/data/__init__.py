"""Data side-chain: preprocessing to ``data.bin`` / ``data.idx.npy``, memory-mapped
datasets with weighted mixing, collators (pretrain / SFT packing / DPO) and the synthetic
token stream. ``get_data_iterator(config)`` returns ``{"train", "eval", "test"}`` iterators of
``{"input_ids", "labels", ...}`` batches.
(Behavioural reference: ironcore/dataloader/__init__.py:14-72.)"""

from __future__ import annotations

import itertools
from typing import Dict, Optional

from .synthetic import SyntheticTokenStream


def get_data_iterator(config, dp_rank: Optional[int] = None, dp_size: Optional[int] = None) -> Dict[str, object]:
    from ..parallel import mesh

    dp_rank = mesh.get_data_parallel_rank() if dp_rank is None else dp_rank
    dp_size = mesh.get_data_parallel_world_size() if dp_size is None else dp_size
    task = str(getattr(config.data, "task_type", "pretrain")).lower()
    has_files = bool(getattr(config.data, "config_path", None))
    if task == "synthetic" or not has_files:
        m = config.model
        vocab = m.vocab_size or config.data.vocab_size
        seed = getattr(config.data, "synthetic_seed", 1234)
        mk = lambda mb, s: SyntheticTokenStream(vocab, m.max_seq_len, mb, seed=s, dp_rank=dp_rank)
        t = config.trainer
        return {
            "train": mk(t.micro_batch_size, seed),
            "eval": mk(t.eval_batch_size or t.micro_batch_size, seed + 1) if t.do_eval else None,
            "test": mk(t.test_batch_size or t.micro_batch_size, seed + 2) if t.do_test else None,
        }
    from .loader import build_file_iterators

    return build_file_iterators(config, dp_rank, dp_size)


__all__ = ["SyntheticTokenStream", "get_data_iterator"]
