"""Rank-0 console logger and scalar loggers with the reference's constructors (``IronCoreLogger(config, ...)``,
``TensorboardLogger(config)``, ``MLFlowLogger(config)``) and method names (reference: ironcore/logger.py:19-210)."""

import logging
from typing import Any, Dict

from ironcore_b200.utils import logging as _l


class LevelFormatter(logging.Formatter):
    """A formatter with one format string per level (``level_formats``: level -> format) and a default."""

    def __init__(self, fmt=None, datefmt=None, level_formats=None):
        super().__init__(fmt=fmt, datefmt=datefmt)
        self._default = logging.Formatter(fmt, datefmt)
        self._by_level = {lvl: logging.Formatter(f, datefmt) for lvl, f in (level_formats or {}).items()}

    def format(self, record):
        return self._by_level.get(record.levelno, self._default).format(record)


def _level_name(level) -> str:
    return logging.getLevelName(level) if isinstance(level, int) else str(level)


class IronCoreLogger(_l.IronCoreLogger):
    """``IronCoreLogger(config, name, level)``: prints on global rank 0 only (errors on every rank)."""

    def __init__(self, config=None, name: str = "ironcore", level=logging.INFO):
        rank = None
        if config is not None and hasattr(config, "parallel"):
            rank = max(int(config.parallel.rank), 0)
        super().__init__(name=name, level=_level_name(level), rank=rank)
        self.logger = self._log

    def set_log_level(self, level):
        self._log.setLevel(level)

    def info(self, message, *a):      # pylint: disable=arguments-renamed
        super().info(message, *a)

    def warning(self, message, *a):   # pylint: disable=arguments-renamed
        super().warning(message, *a)

    def error(self, message, *a):     # pylint: disable=arguments-renamed
        super().error(message, *a)

    def debug(self, message, *a):     # pylint: disable=arguments-renamed
        super().debug(message, *a)

    def log_metrics(self, metrics: Dict[str, Any], msg: str = "evaluation score"):   # pylint: disable=arguments-renamed
        """``metrics``: name -> value, or name -> {column -> value} (one table row per name)."""
        if metrics and all(isinstance(v, dict) for v in metrics.values()):
            cols = []
            for row in metrics.values():
                cols += [c for c in row if c not in cols]
            fmt = lambda v: f"{v:.2f}" if isinstance(v, float) else str(v)
            lines = ["| | " + " | ".join(cols) + " |", "|---|" + "---|" * len(cols)]
            for name, row in metrics.items():
                lines.append(f"| {name} | " + " | ".join(fmt(row.get(c, "")) for c in cols) + " |")
            self.info("%s:\n%s\n", msg, "\n".join(lines))
            return
        super().log_metrics(metrics, title=msg)


class TensorboardLogger(_l.TensorboardLogger):
    """``TensorboardLogger(config)``: writes under ``utils.tensorboard_dir / trainer.model_name`` on rank 0."""

    def __init__(self, config, model_name: str = None):
        if hasattr(config, "utils"):
            self.rank = max(int(config.parallel.rank), 0)
            super().__init__(config.utils.tensorboard_dir, config.trainer.model_name)
        else:   # (log_dir, model_name) as in ironcore_b200
            self.rank = 0
            super().__init__(config, model_name or "model")

    def add_scalar(self, name, value, step):
        if self.rank == 0:
            self.log_metric(name, value, step)

    def add_histogram(self, name, values, step):
        if self.rank == 0:
            self.log_histogram(name, values, step)


class MLFlowLogger(_l.MLFlowLogger):
    """``MLFlowLogger(config)``: active on rank 0 when ``mlflow`` is installed; the run id is kept in
    ``exp_info.json`` so that a resumed job continues its run."""

    def __init__(self, config, *args):
        if hasattr(config, "utils"):
            if int(config.parallel.rank) > 0:
                self.active = False
                return
            super().__init__(config.utils.mlflow_tracking_uri, config.utils.mlflow_experiment_name,
                             config.trainer.model_path, config.trainer.model_name)
        else:   # (tracking_uri, experiment, model_path, run_name) as in ironcore_b200
            super().__init__(config, *args)

    def set_tags(self, tags):
        if self.active:
            self.mlflow.set_tags(tags)

    def set_params(self, params):
        self.set_tags(params)

    def log_metric(self, key, value, step):   # pylint: disable=arguments-renamed
        super().log_metric(key, value, step)

    def log_artifact(self, path):
        if self.active:
            self.mlflow.log_artifact(path)

    def log_artifacts(self, path):
        if self.active:
            self.mlflow.log_artifacts(path)
