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
