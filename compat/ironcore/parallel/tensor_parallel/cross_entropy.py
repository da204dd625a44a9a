"""Reference module path ``ironcore.parallel.tensor_parallel.cross_entropy``."""

from ironcore_b200.parallel.tensor_parallel import vocab_parallel_cross_entropy  # noqa: F401
