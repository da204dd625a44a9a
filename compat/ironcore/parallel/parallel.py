"""Reference module path ``ironcore.parallel.parallel`` (ironcore/parallel/parallel.py)."""

from . import initialize_parallelism, initialize_process  # noqa: F401
