"""``ironcore train`` (reference: ironcore/cli/train.py)."""

from ironcore_b200.cli.train import run_train  # noqa: F401
