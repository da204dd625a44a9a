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
    """Common base of the two linear layers (reference: layers.py:27-60). On its own,
    ``ParallelLinear(config, input_size, output_size, bias)`` is an unsharded ``[in, out]`` weight (and bias)
    without a forward pass, as in the reference."""

    def __init__(self, config=None, input_size: int = None, output_size: int = None, bias: bool = True):
        super().__init__()
        if input_size is None:       # reached through a subclass, which sets everything up itself
            return
        self.config, self.input_size, self.output_size, self.use_bias = config, input_size, output_size, bias
        self.weight = torch.nn.Parameter(torch.empty(input_size, output_size))
        self.bias = torch.nn.Parameter(torch.zeros(output_size)) if bias else None
        self.column_parallel = self.row_parallel = False
        self.concatenated_weights = 1


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

    def init_weight(self):
        """normal(0, init_std) rows, zeros from ``padding_start_idx`` on (this rank's part of them)."""
        std = self.config.init.init_std if self.config is not None else 0.02
        with torch.no_grad():
            self.weight.normal_(0.0, std)
            lo = max(self.padding_start_idx - self.vocab_start, 0)
            if lo < self.rows_per_partition:
                self.weight[lo:].zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # pylint: disable=arguments-differ
        ids = x if x.dim() == 2 else x.reshape(1, -1)
        out = super().forward(ids)
        return out.reshape(*x.shape, self.embedding_dim)


