"""Reference module path ``ironcore.parallel.tensor_parallel.layers``."""

from ironcore_b200.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear,  # noqa: F401
                                                    VocabParallelEmbedding)
