"""Build evaluation tasks from the ``data.eval_datasets`` entries: each ``{"name": task}`` is resolved
to ``ironcore_b200.eval.tasks.<name>`` and the Task subclass found there.
(Behavioural reference: ironcore/eval/evaluator.py:20-64.)"""

from __future__ import annotations

import importlib
from typing import List, Optional

from .tasks.base_task import Task


def get_evaluators(dataset_configs, batch_size: int = 1, num_samples: Optional[int] = None, cache_dir=None,
                   tokenizer=None) -> List[Task]:
    if not dataset_configs:
        return []
    if tokenizer is None:
        from ..global_vars import get_tokenizer

        tokenizer = get_tokenizer()
    if cache_dir is None:
        from ..config.loader import get_dataset_base_dir

        cache_dir = get_dataset_base_dir() / "evaluation_cache"
    tasks = []
    for cfg in dataset_configs:
        if isinstance(cfg, str):
            cfg = {"name": cfg}
        if not isinstance(cfg, dict) or "name" not in cfg:
            continue
        name = str(cfg["name"]).lower()
        try:
            mod = importlib.import_module(f"ironcore_b200.eval.tasks.{name}")
            cls = next(c for c in vars(mod).values() if isinstance(c, type) and issubclass(c, Task) and c is not Task)
        except (ImportError, StopIteration):
            print(f"Evaluator for task '{name}' could not be loaded.")
            continue
        tasks.append(cls(tokenizer, batch_size or 1, cfg.get("samples", num_samples), cache_dir=cache_dir))
    return tasks
