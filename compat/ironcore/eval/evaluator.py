"""Evaluator registry (reference: ironcore/eval/evaluator.py:20-64)."""

from ironcore_b200.eval.evaluator import get_evaluators  # noqa: F401
