"""Dataset YAML schema: a list of dataset sources (name, source, task type, mixing ratio, columns)
plus tokenizer, sequence length, split ratios and output directories.
(Behavioural reference: ironcore/dataloader/data_config.py:15-231; ``max_seq_len`` follows
``seq_length`` here instead of staying at 1024.)"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Union

from ..config.loader import load_yaml_config

TASK_TYPES = ("pretrain", "sft", "dpo")


@dataclass
class DatasetConfig:
    name: str
    source: str
    task_type: str = "pretrain"
    ratio: float = 1.0
    split: Optional[str] = "train"
    subset: Optional[str] = None
    text_column: str = "text"
    messages_column: str = "messages"
    chosen_column: str = "chosen"
    rejected_column: str = "rejected"
    chat_template: Optional[str] = None
    max_samples: Optional[int] = None
    output_path: Optional[Path] = None

    def __post_init__(self):
        if self.ratio <= 0:
            raise ValueError(f"Dataset {self.name}: ratio must be positive, got {self.ratio}")
        if self.task_type not in TASK_TYPES:
            raise ValueError(f"Dataset {self.name}: invalid task_type {self.task_type}")

    @classmethod
    def from_dict(cls, d: Dict) -> "DatasetConfig":
        d = dict(d)
        if "dataset_path" in d and "source" not in d:
            d["source"] = d.pop("dataset_path")
        d.pop("dataset_path", None)
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})


@dataclass
class UniversalDataConfig:
    datasets: List[DatasetConfig]
    eval_datasets: List[DatasetConfig] = field(default_factory=list)
    test_datasets: List[DatasetConfig] = field(default_factory=list)
    vocab_name_or_path: str = "gpt2"
    tokenizer_type: str = "bbpe"
    seq_length: int = 1024
    max_seq_len: Optional[int] = None
    splits: List[float] = field(default_factory=lambda: [0.99, 0.01, 0.0])
    pad_token_id: Optional[int] = None
    preprocessed_dir: Path = Path("./data/preprocessed")
    cache_dir: Path = Path("./data/cache")
    num_workers: int = 4
    preprocessing: Dict = field(default_factory=dict)

    def __post_init__(self):
        self.preprocessed_dir = Path(self.preprocessed_dir)
        self.cache_dir = Path(self.cache_dir)
        if abs(sum(self.splits) - 1.0) > 1e-6:
            raise ValueError(f"Splits must sum to 1.0, got {sum(self.splits)}")
        if not self.datasets:
            raise ValueError("At least one dataset must be specified")
        if self.max_seq_len is None:
            self.max_seq_len = self.seq_length
        for ds in self.all_datasets():
            if ds.output_path is None:
                ds.output_path = self.output_dir(ds)

    def all_datasets(self) -> List[DatasetConfig]:
        return list(self.datasets) + list(self.eval_datasets) + list(self.test_datasets)

    def output_dir(self, ds: DatasetConfig) -> Path:
        return self.preprocessed_dir / ds.name / ds.task_type

    def get_dataset_output_path(self, dataset: DatasetConfig) -> Path:
        """Directory of a dataset's ``data.bin`` / ``data.idx.npy`` (created when missing)."""
        out = Path(dataset.output_path) if dataset.output_path else self.output_dir(dataset)
        out.mkdir(parents=True, exist_ok=True)
        return out

    @classmethod
    def from_yaml(cls, path: Union[str, Path]) -> "UniversalDataConfig":
        return cls.from_dict(load_yaml_config(path, merge_lists=False))

    @classmethod
    def from_dict(cls, doc: Dict) -> "UniversalDataConfig":
        def parse(key_a, key_b=None):
            raw = doc.get(key_a) or (doc.get(key_b) if key_b else None) or []
            if isinstance(raw, dict):  # list of single-key dicts was merged by the YAML helper
                raw = [dict(v, name=v.get("name", k)) if isinstance(v, dict) else v for k, v in raw.items()]
            return [DatasetConfig.from_dict(d) for d in raw]

        kw = {k: doc[k] for k in ("vocab_name_or_path", "tokenizer_type", "seq_length", "max_seq_len", "splits",
                                  "pad_token_id", "preprocessed_dir", "cache_dir", "num_workers", "preprocessing")
              if k in doc}
        return cls(datasets=parse("train_datasets", "datasets"), eval_datasets=parse("eval_datasets"),
                   test_datasets=parse("test_datasets"), **kw)


def load_data_config(config_path: Union[str, Path]) -> UniversalDataConfig:
    return UniversalDataConfig.from_yaml(config_path)


DataConfig = UniversalDataConfig     # the reference's alias (ironcore/dataloader/data_config.py:231)
