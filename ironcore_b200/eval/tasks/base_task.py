"""Evaluation task interface: ``Task.process(model) -> {"metric": name, "score": value}``.
(Behavioural reference: ironcore/eval/tasks/base_task.py:21-89.)"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional


class Task:
    name = "task"
    metric = "accuracy"

    def __init__(self, tokenizer, batch_size: int = 1, num_samples: Optional[int] = None, cache_dir=None,
                 examples: Optional[List[dict]] = None):
        self.tokenizer = tokenizer
        self.batch_size = max(int(batch_size or 1), 1)
        self.num_samples = num_samples
        self.cache_dir = cache_dir
        self._examples = examples

    @property
    def task_name(self) -> str:
        return self.name

    def load_examples(self) -> Iterable[dict]:
        raise NotImplementedError

    def examples(self) -> List[dict]:
        if self._examples is None:
            self._examples = list(self.load_examples())
        ex = self._examples
        return ex[: self.num_samples] if self.num_samples else ex

    def process(self, model) -> Dict[str, float]:
        raise NotImplementedError
