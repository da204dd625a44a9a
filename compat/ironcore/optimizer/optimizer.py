"""AdamW (reference: ironcore/optimizer/optimizer.py:16-120)."""

from ironcore_b200.optim.adam import AdamWOptimizer  # noqa: F401
