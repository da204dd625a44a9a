"""Process-wide singletons: config, logger, metric sinks, timer, tokenizer.
(Behavioural reference: ironcore/global_vars.py:21-128.)"""

from __future__ import annotations

from typing import Dict, Optional

from .tokenizer import build_tokenizer
from .utils.logging import IronCoreLogger, MLFlowLogger, TensorboardLogger
from .utils.timers import Timer


class GlobalStates:
    def __init__(self, config=None, tokenizer=None):
        self.config = None
        self.logger: Optional[IronCoreLogger] = None
        self.tb: Optional[TensorboardLogger] = None
        self.mlflow: Optional[MLFlowLogger] = None
        self.timer: Optional[Timer] = None
        self.tokenizer = None
        if config is not None:
            self.setup(config, tokenizer)

    def setup(self, config, tokenizer=None) -> "GlobalStates":
        """Create the logger, timer, tokenizer and metric sinks for ``config``; records the tokenizer's vocabulary
        sizes and special ids in the model config."""
        self.config = config
        self.logger = IronCoreLogger(level=config.utils.log_level, rank=max(config.parallel.rank, 0))
        self.timer = Timer()
        self.tokenizer = tokenizer if tokenizer is not None else build_tokenizer(config)
        m = config.model
        m.vocab_size = self.tokenizer.vocab_size
        m.padded_vocab_size = self.tokenizer.padded_vocab_size
        m.eod_token_id = self.tokenizer.eod_token_id
        m.pad_token_id = self.tokenizer.pad_token_id
        rank0 = max(config.parallel.rank, 0) == 0
        if rank0 and config.utils.tensorboard_dir:
            self.tb = TensorboardLogger(config.utils.tensorboard_dir, config.trainer.model_name)
        if rank0 and config.utils.mlflow_tracking_uri:
            self.mlflow = MLFlowLogger(config.utils.mlflow_tracking_uri, config.utils.mlflow_experiment_name,
                                       config.trainer.model_path, config.trainer.model_name)
        return self

    # accessors under the reference's method names (ironcore/global_vars.py:41-57)
    def get_config(self):
        return self.config

    def get_logger(self):
        return get_logger()

    def get_tokenizer(self):
        return self.tokenizer

    def cleanup(self):
        global_states_cleanup()


_G = GlobalStates()


def set_global_states(config, tokenizer=None) -> GlobalStates:
    """Create the singletons once; records the tokenizer's vocabulary sizes in the model config."""
    return _G.setup(config, tokenizer)


def get_global_states() -> GlobalStates:
    return _G


def get_config():
    return _G.config


def get_logger() -> IronCoreLogger:
    if _G.logger is None:
        _G.logger = IronCoreLogger()
    return _G.logger


def get_timer() -> Timer:
    if _G.timer is None:
        _G.timer = Timer()
    return _G.timer


def get_tokenizer():
    return _G.tokenizer


def log_metric(name: str, value, step: int):
    for sink in (_G.tb, _G.mlflow):
        if sink is not None:
            sink.log_metric(name, value, step)


def log_metrics(metrics: Dict[str, float], step: int):
    for k, v in metrics.items():
        log_metric(k, v, step)


def log_histogram(name: str, values, step: int):
    if _G.tb is not None:
        _G.tb.log_histogram(name, values, step)


def global_states_cleanup():
    for sink in (_G.tb, _G.mlflow):
        if sink is not None:
            sink.close()
    _G.tb = _G.mlflow = None
