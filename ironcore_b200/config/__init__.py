"""Hierarchical configuration (groups: model, init, optim, data, parallel, trainer,
operation, utils, rl) with YAML, command-line and environment sources."""

from .loader import (
    apply_cli_overrides,
    apply_env_ranks,
    apply_yaml,
    build_arg_parser,
    data_parallel_size,
    default_config,
    get_dataset_base_dir,
    load_config,
    load_trainer_config,
    load_yaml_config,
    validate_config,
)
from .schema import (
    GROUPS,
    BaseConfig,
    DataConfig,
    InitConfig,
    MainConfig,
    ModelConfig,
    MoEConfig,
    OperationConfig,
    OptimConfig,
    ParallelConfig,
    PositionalEmbeddingConfig,
    RLConfig,
    TrainerConfig,
    UtilsConfig,
)

__all__ = [
    "GROUPS", "BaseConfig", "DataConfig", "InitConfig", "MainConfig", "ModelConfig", "MoEConfig", "OperationConfig",
    "OptimConfig", "ParallelConfig", "PositionalEmbeddingConfig", "RLConfig", "TrainerConfig", "UtilsConfig",
    "apply_cli_overrides", "apply_env_ranks", "apply_yaml", "build_arg_parser", "data_parallel_size",
    "default_config", "get_dataset_base_dir", "load_config", "load_trainer_config", "load_yaml_config",
    "validate_config",
]
