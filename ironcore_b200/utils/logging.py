"""Rank-0 console logger, metric table, TensorBoard and MLflow sinks.
(Behavioural reference: ironcore/logger.py:34-210.)"""

from __future__ import annotations

import json
import logging
import os
import sys
from pathlib import Path
from typing import Dict, Optional


class IronCoreLogger:
    """Console logger that prints on global rank 0 only (other ranks log errors)."""

    def __init__(self, name: str = "ironcore_b200", level: str = "INFO", rank: Optional[int] = None):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self._log = logging.getLogger(f"{name}.{self.rank}")
        self._log.setLevel(getattr(logging, str(level).upper(), logging.INFO))
        self._log.propagate = False
        if not self._log.handlers:
            h = logging.StreamHandler(sys.stdout)
            h.setFormatter(logging.Formatter("[%(asctime)s][%(levelname)s] %(message)s", "%Y-%m-%d %H:%M:%S"))
            self._log.addHandler(h)

    def _emit(self, level, msg, *a):
        if self.rank == 0 or level >= logging.ERROR:
            self._log.log(level, msg, *a, stacklevel=3)

    def debug(self, msg, *a):
        self._emit(logging.DEBUG, msg, *a)

    def info(self, msg, *a):
        self._emit(logging.INFO, msg, *a)

    def warning(self, msg, *a):
        self._emit(logging.WARNING, msg, *a)

    def error(self, msg, *a):
        self._emit(logging.ERROR, msg, *a)

    def log_metrics(self, metrics: Dict[str, float], title: str = "metrics"):
        """Markdown table of name/value pairs."""
        if self.rank != 0:
            return
        width = max([len(k) for k in metrics] + [6])
        lines = [f"| {'metric'.ljust(width)} | value |", f"|{'-' * (width + 2)}|-------|"]
        for k, v in metrics.items():
            val = f"{v:.6g}" if isinstance(v, (int, float)) else str(v)
            lines.append(f"| {k.ljust(width)} | {val} |")
        self.info("%s\n%s", title, "\n".join(lines))


class TensorboardLogger:
    def __init__(self, log_dir: str, model_name: str = "model"):
        self.writer = None
        try:
            from torch.utils.tensorboard import SummaryWriter

            self.writer = SummaryWriter(log_dir=str(Path(log_dir) / model_name))
        except Exception:  # tensorboard not installed: keep a JSONL fallback next to it
            Path(log_dir, model_name).mkdir(parents=True, exist_ok=True)
            self._jsonl = open(Path(log_dir) / model_name / "scalars.jsonl", "a")

    def log_metric(self, name, value, step):
        if self.writer is not None:
            self.writer.add_scalar(name, value, step)
        else:
            self._jsonl.write(json.dumps({"name": name, "value": float(value), "step": int(step)}) + "\n")
            self._jsonl.flush()

    def log_histogram(self, name, values, step):
        if self.writer is not None:
            self.writer.add_histogram(name, values, step)

    def close(self):
        if self.writer is not None:
            self.writer.close()
        elif getattr(self, "_jsonl", None) is not None:
            self._jsonl.close()


class MLFlowLogger:
    """MLflow sink; the run id is persisted in ``exp_info.json`` under the model path so a
    resumed job continues the same run. A no-op when mlflow is not installed."""

    def __init__(self, tracking_uri: str, experiment: Optional[str], model_path: str, run_name: str = "model"):
        self.active = False
        try:
            import mlflow
        except Exception:
            return
        self.mlflow = mlflow
        mlflow.set_tracking_uri(tracking_uri)
        if experiment:
            mlflow.set_experiment(experiment)
        info = Path(model_path or ".") / "exp_info.json"
        run_id = None
        if info.exists():
            run_id = json.loads(info.read_text()).get("run_id")
        run = mlflow.start_run(run_id=run_id, run_name=run_name)
        info.parent.mkdir(parents=True, exist_ok=True)
        info.write_text(json.dumps({"run_id": run.info.run_id}))
        self.active = True

    def log_metric(self, name, value, step):
        if self.active:
            self.mlflow.log_metric(name, float(value), step=int(step))

    def log_params(self, params: dict):
        if self.active:
            self.mlflow.log_params(params)

    def close(self):
        if self.active:
            self.mlflow.end_run()
