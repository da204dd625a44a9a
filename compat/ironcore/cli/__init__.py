"""Sub-command handlers (reference: ironcore/cli/{train,preprocess,inspect}.py)."""

from .inspect import run_inspect  # noqa: F401
from ironcore_b200.cli.preprocess import run_preprocess  # noqa: F401
from ironcore_b200.cli.train import run_train  # noqa: F401
