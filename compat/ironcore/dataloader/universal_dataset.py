"""Binary datasets and weighted mixing with the reference's constructors
(reference: ironcore/dataloader/universal_dataset.py:20-390)."""

from pathlib import Path

from ironcore_b200.data import dataset as _ds


class BinaryDataset(_ds.BinaryDataset):
    """``BinaryDataset(bin_path, idx_path)`` (both files of one dataset directory) or ``BinaryDataset(directory)``."""

    def __init__(self, bin_path, idx_path=None):
        p = Path(bin_path)
        super().__init__(p if p.is_dir() else p.parent)
        self.bin_path, self.idx_path = p, Path(idx_path) if idx_path is not None else None
        self.metadata, self.data = self.index, self.tokens

    def total_tokens(self) -> int:
        return self.num_tokens

    def __getitem__(self, idx: int):
        s = self.sample(idx)
        meta = {k: s[k] for k in ("type", "group_id", "mask_ranges")}
        meta["length"] = len(s["tokens"])
        return {"token_ids": s["tokens"], "metadata": meta}


class WeightedMixingDataset(_ds.WeightedMixingDataset):
    """``WeightedMixingDataset(data_config, mode, seed, split)``; this rank's share of the data follows the
    data-parallel layout of the initialised mesh (rank 0 of 1 without one)."""

    def __init__(self, data_config, mode: str = "pretrain", seed: int = 1337, split: str = "train", dp_rank=None,
                 dp_size=None, epochs=None, seq_len=None):
        from ironcore_b200.parallel import mesh

        super().__init__(seq_len=seq_len or data_config.max_seq_len, seed=seed, epochs=epochs,
                         dp_rank=mesh.get_data_parallel_rank() if dp_rank is None else dp_rank,
                         dp_size=mesh.get_data_parallel_world_size() if dp_size is None else dp_size,
                         **self.sources_of(data_config, mode, split))
        self.config, self.max_seq_len = data_config, self.seq_len
        self.datasets = self.sets
