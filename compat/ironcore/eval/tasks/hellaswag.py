"""HellaSwag (reference: ironcore/eval/tasks/hellaswag.py)."""

from ironcore_b200.eval.tasks.hellaswag import HellaSwag  # noqa: F401
