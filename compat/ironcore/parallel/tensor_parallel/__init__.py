"""Tensor-parallel layers, collectives and loss (reference: ironcore/parallel/tensor_parallel/__init__.py)."""

from .cross_entropy import vocab_parallel_cross_entropy  # noqa: F401
from .layers import ColumnParallelLinear, ParallelLinear, RowParallelLinear, VocabParallelEmbedding  # noqa: F401

from .comm import (copy_inputs_to_model_parallel_workers, gather_from_model_parallel_workers,  # noqa: F401
                   reduce_inputs_from_model_parallel_workers, scatter_input_to_model_parallel_workers,
                   split_to_model_parallel_workers)

__all__ = ["ColumnParallelLinear", "RowParallelLinear", "VocabParallelEmbedding",
           "copy_inputs_to_model_parallel_workers", "reduce_inputs_from_model_parallel_workers",
           "scatter_input_to_model_parallel_workers", "vocab_parallel_cross_entropy"]
