"""Task base class with the reference's constructor (reference: ironcore/eval/tasks/base_task.py:21-89)."""

from ironcore_b200.eval.tasks import base_task as _base


class Task(_base.Task):
    """``Task(task_name, split_name, tokenizer, batch_size, num_samples, cache_dir)``: subclasses provide
    ``load_examples()`` (the ``split_name`` split of the ``task_name`` dataset) and ``process(model)``."""

    def __init__(self, task_name: str, split_name: str, tokenizer, batch_size: int = 1, num_samples: int = None,
                 cache_dir=None, examples=None):
        super().__init__(tokenizer, batch_size, num_samples, cache_dir, examples)
        self.name = task_name
        self.split_name = split_name
