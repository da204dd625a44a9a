"""Evaluation tasks (reference: ironcore/eval/tasks/)."""

from ironcore_b200.eval.tasks.base_task import Task  # noqa: F401
from ironcore_b200.eval.tasks.hellaswag import HellaSwag  # noqa: F401
