from .evaluator import get_evaluators
from .tasks.base_task import Task

__all__ = ["Task", "get_evaluators"]
