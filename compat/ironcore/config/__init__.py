"""Configuration groups and loaders under the reference's names (ironcore/config/__init__.py:33-515).
``_config_validation`` is ``validate_config``; ``_load_config_from_yaml(config, args)`` reads
``args.config`` (or ``args.config_path``) like the reference's loader."""

from ironcore_b200.config import (BaseConfig, DataConfig, InitConfig, MainConfig, ModelConfig,  # noqa: F401
                                  OperationConfig, OptimConfig, ParallelConfig, TrainerConfig, UtilsConfig,
                                  apply_yaml, build_arg_parser, default_config, load_trainer_config,
                                  load_yaml_config, validate_config)
from ironcore_b200.config.schema import PositionalEmbeddingConfig  # noqa: F401

_config_validation = validate_config


def _load_config_from_yaml(config, args):
    path = getattr(args, "config", None) or getattr(args, "config_path", None)
    return apply_yaml(config, path)


def parse_args(argv=None):
    return build_arg_parser().parse_args(argv)


def print_args(config):
    """Print every field of every configuration group as ``group.field: value``."""
    from dataclasses import fields

    for group in fields(config):
        node = getattr(config, group.name)
        for f in fields(node):
            print(f"{group.name}.{f.name}: {getattr(node, f.name)}")


def load_data_config(config, datasets):
    """``{dataset name or path: {ratio, samples, subgroup}}`` -> list of ``{name, dataset_path, ratio, samples}``.
    A name is looked up under ``$PROCESSED_DATA_PATH`` (or ``$DATASET_DIR/preprocessed_corpus``) /
    ``<data.name>`` / ``<name>[_<subgroup>]``; a path whose ``.bin`` file exists is taken as it is.
    (Reference: ironcore/config/__init__.py:172-215.)"""
    import os
    from pathlib import Path

    out = []
    for key, spec in (datasets or {}).items():
        spec = spec or {}
        item = {}
        if Path(key).with_suffix(".bin").exists():
            item["name"], item["dataset_path"] = os.path.basename(key), key
        else:
            base = os.environ.get("PROCESSED_DATA_PATH") or Path(os.environ.get("DATASET_DIR", ".")) / "preprocessed_corpus"
            name = f"{key}_{spec['subgroup']}" if spec.get("subgroup") else key
            item["name"] = name
            item["dataset_path"] = Path(base) / str(getattr(config.data, "name", "") or "") / name
        if "ratio" in spec:
            item["ratio"] = spec.get("ratio", 1.0)
        if "samples" in spec:
            item["samples"] = spec.get("samples")
        out.append(item)
    return out
