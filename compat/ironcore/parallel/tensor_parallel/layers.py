"""Tensor-parallel layers with the reference's constructor and call conventions
(reference: ironcore/parallel/tensor_parallel/layers.py:27-262): the configuration object comes first, and inputs
may carry any number of leading dimensions (``[b, s, h]`` in the reference's model). The work is done by the
``ironcore_b200`` layers; weights keep that package's ``[in, out]`` orientation."""

from __future__ import annotations

import torch

from ironcore_b200.parallel import tensor_parallel as _tp


def _flat(x: torch.Tensor):
    return x.reshape(-1, x.shape[-1]), x.shape[:-1]


class ParallelLinear(torch.nn.Module):
    """Common base of the two linear layers (reference: layers.py:27-60); it carries no behaviour here."""


class ColumnParallelLinear(_tp.ColumnParallelLinear, ParallelLinear):
    def __init__(self, config, input_size: int, output_size: int, bias: bool = True, gather_output: bool = False,
                 concatenated_weights=None):
        super().__init__(input_size, output_size, bias=bias, gather_output=gather_output,
                         concatenated_weights=concatenated_weights or 1)
        self.config = config
        self.input_size, self.output_size = input_size, output_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # pylint: disable=arguments-differ
        flat, lead = _flat(x)
        return super().forward(flat).reshape(*lead, -1)


class RowParallelLinear(_tp.RowParallelLinear, ParallelLinear):
    def __init__(self, config, input_size: int, output_size: int, bias: bool = True, input_is_parallel: bool = True):
        super().__init__(input_size, output_size, bias=bias, input_is_parallel=input_is_parallel)
        self.config = config
        self.input_size, self.output_size = input_size, output_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # pylint: disable=arguments-differ
        flat, lead = _flat(x)
        return super().forward(flat).reshape(*lead, -1)


class VocabParallelEmbedding(_tp.VocabParallelEmbedding):
    """``forward(ids [b, s]) -> [b, s, d]``. ``parallel_input`` / ``parallel_output`` are accepted for the
    reference's signature; the table is always sharded by vocabulary rows and the output is always the reduced
    (complete) embedding."""

    def __init__(self, config, input_dim: int, embedding_dim: int, padding_start_idx=None, parallel_input: bool = True,
                 parallel_output: bool = False):
        super().__init__(input_dim, embedding_dim, padding_start_idx=padding_start_idx)
        self.config = config
        self.parallel_input, self.parallel_output = parallel_input, parallel_output

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # pylint: disable=arguments-differ
        ids = x if x.dim() == 2 else x.reshape(1, -1)
        out = super().forward(ids)
        return out.reshape(*x.shape, self.embedding_dim)


