"""Task base class (reference: ironcore/eval/tasks/base_task.py)."""

from ironcore_b200.eval.tasks.base_task import Task  # noqa: F401
