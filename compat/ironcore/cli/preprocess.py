"""``ironcore preprocess`` (reference: ironcore/cli/preprocess.py:10-75)."""

from ironcore_b200.cli.preprocess import run_preprocess  # noqa: F401
