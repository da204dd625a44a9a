"""Megatron-style tensor-parallel layers with optional sequence parallelism.

Weights are stored ``[in, out]`` and applied as ``x @ W``.

* ``ColumnParallelLinear``: output features sharded over the TP group. Input is either
  replicated (identity forward / all-reduce backward) or, with sequence parallelism, a
  token shard that is all-gathered in forward and whose gradient is reduce-scattered.
* ``RowParallelLinear``: input features sharded; the partial products are all-reduced,
  or reduce-scattered onto token shards under sequence parallelism.
* ``VocabParallelEmbedding``: vocabulary rows sharded; foreign ids contribute zeros and
  the partial embeddings are summed (reduce-scattered under sequence parallelism).
* ``vocab_parallel_cross_entropy``: loss over vocab-sharded logits with three scalar
  exchanges per token instead of gathering logits.

On CUDA (16-bit dtypes) the GEMMs are the tcgen05 kernel and, when a symmetric-memory
workspace is attached (see ``fused_comm``), gather+GEMM and GEMM+reduce-scatter run as
single fused kernels; the ``torch.distributed`` path below is the baseline and oracle.
(Behavioural reference: ironcore/parallel/tensor_parallel/layers.py:25-263,
ironcore/parallel/tensor_parallel/cross_entropy.py:35-155.)
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as OF
from . import collectives as C
from . import mesh


def divide(a: int, b: int) -> int:
    if a % b != 0:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def _accept_full_tensors(module: nn.Module) -> None:
    """Let ``load_state_dict`` take the unsharded (tensor-parallel size 1) tensor for a sharded parameter of
    ``module``: an entry whose shape is the full shape is replaced by this rank's slice before it is copied, so a
    plain ``state_dict()`` of a single-rank model loads into any tensor-parallel size."""

    def hook(state_dict, prefix, *_unused):
        if module.tp_size == 1:
            return
        for name, p in module._parameters.items():   # pylint: disable=protected-access
            dim = getattr(p, "tp_shard_dim", None) if p is not None else None
            t = state_dict.get(prefix + name)
            if dim is None or t is None or t.dim() != p.dim() or t.shape == p.shape or p.numel() == 0:
                continue
            full = list(p.shape)
            full[dim] *= module.tp_size
            if list(t.shape) == full:
                state_dict[prefix + name] = shard_tensor(t, dim, getattr(p, "tp_parts", 1), C._rank(module.tp_group),
                                                         module.tp_size)

    module._register_load_state_dict_pre_hook(hook)   # pylint: disable=protected-access


class ColumnParallelLinear(nn.Module):
    """y_local = gather(x) @ W[:, shard] + b[shard].

    ``concatenated_weights`` = number of equal logical matrices fused along the output
    dim (2 for K|V or gate|up); each is sharded separately so that a rank holds matching
    slices of every part.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = False,
                 concatenated_weights=1, dtype=None, device=None, tp_group="default"):
        super().__init__()
        self.tp_group = mesh.get_tensor_model_parallel_group() if tp_group == "default" else tp_group
        self.tp_size = C._size(self.tp_group)
        self.in_features = in_features
        self.out_features = out_features
        self.out_per_partition = divide(out_features, self.tp_size)
        self.gather_output = gather_output
        self.column_parallel = True
        self.concatenated_weights = concatenated_weights
        self.sequence_parallel = mesh.sequence_parallel_enabled() and self.tp_size > 1
        self.weight = nn.Parameter(torch.empty(in_features, self.out_per_partition, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(self.out_per_partition, dtype=dtype, device=device)) if bias else None
        self.weight.tp_shard_dim = 1
        self.weight.tp_parts = concatenated_weights
        if self.bias is not None:
            self.bias.tp_shard_dim = 0
            self.bias.tp_parts = concatenated_weights
        self.fused = None        # optional fused gather+GEMM workspace
        self.gather_slot = None  # this call site's persistent gathered buffer inside that workspace
        _accept_full_tensors(self)

    def gather_target(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """This rank's rows of the gather slot, when ``self(x')`` for an ``x'`` shaped like ``x`` will run the
        fused gather: the producer of ``x'`` can write there directly and spare the copy into the slot."""
        ws, slot = self.fused, self.gather_slot
        if ws is None or slot is None or not self.sequence_parallel or not OF.use_native(x):
            return None
        if x.dim() != 2 or x.shape[0] != ws.rows or x.shape[1] != ws.width or x.dtype != ws.dtype:
            return None
        return slot.local

    def forward(self, x: torch.Tensor, pregathered: bool = False) -> torch.Tensor:
        """``pregathered``: ``x`` is this rank's part of ``gather_slot`` and every rank's part was written
        there by the kernel that produced it (``RowParallelLinear.forward_norm``): nothing is pushed."""
        if pregathered and (self.fused is None or self.gather_slot is None):
            raise RuntimeError("a pregathered input needs the fused workspace and a gather slot")
        if self.tp_size > 1:
            if self.sequence_parallel:
                if self.fused is not None and OF.use_native(x) and x.dim() == 2 and x.shape[0] == self.fused.rows:
                    y = self.fused.allgather_linear(x, self.weight, self.bias, self.gather_slot, pregathered)
                    return C.gather_last_dim(y, self.tp_group) if self.gather_output else y
                x = C.gather_from_sp(x, self.tp_group)
            else:
                x = C.copy_to_tp(x, self.tp_group)
        y = OF.linear(x, self.weight, self.bias)
        if self.gather_output and self.tp_size > 1:
            y = C.gather_last_dim(y, self.tp_group)
        return y

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features} (/{self.tp_size}), parts={self.concatenated_weights}"


class RowParallelLinear(nn.Module):
    """y = reduce(x_local @ W[shard, :]) + b."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, input_is_parallel: bool = True,
                 dtype=None, device=None, tp_group="default"):
        super().__init__()
        self.tp_group = mesh.get_tensor_model_parallel_group() if tp_group == "default" else tp_group
        self.tp_size = C._size(self.tp_group)
        self.in_features = in_features
        self.out_features = out_features
        self.in_per_partition = divide(in_features, self.tp_size)
        self.input_is_parallel = input_is_parallel
        self.row_parallel = True
        self.sequence_parallel = mesh.sequence_parallel_enabled() and self.tp_size > 1
        self.weight = nn.Parameter(torch.empty(self.in_per_partition, out_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.weight.tp_shard_dim = 0
        self.weight.tp_parts = 1
        if self.bias is not None:
            # replicated parameter that sees different tokens per rank under sequence parallelism
            self.bias.sp_replicated = True
        self.fused = None
        _accept_full_tensors(self)

    def can_fuse_norm(self, x: torch.Tensor, norm, consumer) -> bool:
        """Whether ``forward_norm`` can run as one kernel: fused workspace on both ends, RMSNorm without
        bias, a row width the producer kernel supports."""
        ws = self.fused
        return (ws is not None and self.sequence_parallel and getattr(consumer, "fused", None) is ws
                and getattr(consumer, "gather_slot", None) is not None and ws.norm_fusable
                and getattr(norm, "rms", False) and norm.layernorm.bias is None and OF.use_native(x)
                and x.dim() == 2 and x.shape[0] == ws.tokens and self.input_is_parallel
                and not getattr(consumer, "gather_output", False))

    def forward_norm(self, x: torch.Tensor, residual: Optional[torch.Tensor], norm, consumer):
        """``h = self(x, residual)`` followed by ``norm(h)``, with the normalised rows delivered into the
        gather slot of ``consumer`` (the column-parallel linear that reads them next) on every rank by the
        same kernel that reduces the partial products. Returns ``(h, normed)``; pass ``normed`` to
        ``consumer(normed, pregathered=True)``. Callers check ``can_fuse_norm`` first."""
        return self.fused.linear_reduce_scatter_norm(x, self.weight, self.bias, residual, norm.layernorm.weight,
                                                     norm.eps, norm.weight_offset, consumer.gather_slot)

    def forward_norm_linear(self, x: torch.Tensor, residual: Optional[torch.Tensor], norm, consumer):
        """``h = self(x, residual)``; ``y = consumer(norm(h))`` with the whole boundary fused in both
        directions (see ``fused_comm._RowNormColumn``). Returns ``(h, y)``. Callers check ``can_fuse_norm``."""
        return self.fused.row_norm_column(x, self.weight, self.bias, residual, norm.layernorm.weight, norm.eps,
                                          norm.weight_offset, consumer.weight, consumer.bias, consumer.gather_slot)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual`` (optional, already in the output layout) is added after the reduction."""
        if self.tp_size == 1:
            return OF.linear(x, self.weight, self.bias, residual)
        if not self.input_is_parallel:
            x = C.scatter_last_dim(x, self.tp_group)
        if self.sequence_parallel and self.fused is not None and OF.use_native(x) and x.dim() == 2 \
                and x.shape[0] == self.fused.tokens:
            return self.fused.linear_reduce_scatter(x, self.weight, self.bias, residual)
        y = OF.linear(x, self.weight, None)
        if self.sequence_parallel:
            y = C.reduce_scatter_to_sp(y, self.tp_group)
        else:
            y = C.reduce_from_tp(y, self.tp_group)
        if self.bias is not None:
            y = y + self.bias
        if residual is not None:
            y = y + residual
        return y

    def extra_repr(self):
        return f"in={self.in_features} (/{self.tp_size}), out={self.out_features}"


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded by vocabulary rows. ``padding_start_idx`` = first padded
    (never used) row of the full table; those rows are zero-initialised."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_start_idx: Optional[int] = None, dtype=None,
                 device=None, tp_group="default"):
        super().__init__()
        self.tp_group = mesh.get_tensor_model_parallel_group() if tp_group == "default" else tp_group
        self.tp_size = C._size(self.tp_group)
        self.tp_rank = C._rank(self.tp_group)
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.rows_per_partition = divide(num_embeddings, self.tp_size)
        self.vocab_start = self.tp_rank * self.rows_per_partition
        self.vocab_end = self.vocab_start + self.rows_per_partition
        self.padding_start_idx = padding_start_idx if padding_start_idx is not None else num_embeddings
        self.row_parallel = True
        self.sequence_parallel = mesh.sequence_parallel_enabled() and self.tp_size > 1
        self.weight = nn.Parameter(torch.empty(self.rows_per_partition, embedding_dim, dtype=dtype, device=device))
        self.weight.tp_shard_dim = 0
        self.weight.tp_parts = 1
        _accept_full_tensors(self)

    def forward(self, ids: torch.Tensor, pos_table: Optional[torch.Tensor] = None,
                pos_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [B, S] -> [B*S, D] token-major (a token shard under sequence parallelism)."""
        if self.tp_size == 1:
            out = OF.embedding(ids, self.weight, pos_table=pos_table, pos_ids=pos_ids)
            return out.reshape(-1, self.embedding_dim)
        # the position table is replicated: only one rank may add it before the sum
        pt = pos_table if self.tp_rank == 0 else None
        out = OF.embedding(ids, self.weight, vocab_start=self.vocab_start, pos_table=pt, pos_ids=pos_ids)
        if pos_table is not None and self.tp_rank != 0:
            out = out + 0.0 * pos_table.sum()  # keep the parameter in the graph on every rank
        out = out.reshape(-1, self.embedding_dim)
        if self.sequence_parallel:
            return C.reduce_scatter_to_sp(out, self.tp_group)
        return C.reduce_from_tp(out, self.tp_group)


def vocab_parallel_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab_size: Optional[int] = None,
                                 tp_group="default") -> torch.Tensor:
    """Per-token loss for logits [T, V/t] sharded over the TP group. ``vocab_size`` = number
    of real (unpadded) vocabulary entries; padded columns are excluded from the softmax."""
    group = mesh.get_tensor_model_parallel_group() if tp_group == "default" else tp_group
    n, r = C._size(group), C._rank(group)
    v_local = logits.shape[-1]
    start = r * v_local
    valid = v_local
    if vocab_size is not None:
        valid = max(0, min(v_local, vocab_size - start))
    flat = logits.reshape(-1, v_local)
    loss = OF.cross_entropy(flat, targets.reshape(-1), vocab_start=start, vocab_valid=valid,
                            group=group if n > 1 else None)
    return loss.view(targets.shape)


def init_linear_weight_(param: torch.Tensor, full_shape, std: float, shard_dim: Optional[int], parts: int,
                        tp_rank: int, tp_size: int, xavier: bool = False, generator=None,
                        valid: Optional[tuple] = None) -> None:
    """Initialise a (possibly TP-sharded) weight so that TP=k equals the shards of the TP=1
    tensor: draw the full matrix from the shared RNG stream, keep this rank's slice.
    ``valid`` = (dim, n): only the first ``n`` entries along ``dim`` are drawn, the rest (vocabulary padding, whose
    amount depends on the TP size) are zeros, so that the stream of random numbers does not depend on the padding."""
    drawn = list(full_shape)
    if valid is not None:
        drawn[valid[0]] = min(int(valid[1]), drawn[valid[0]])
    full = torch.empty(drawn, dtype=torch.float32)
    if xavier:
        bound = math.sqrt(6.0 / (drawn[0] + drawn[1]))
        full.uniform_(-bound, bound, generator=generator)
    else:
        full.normal_(mean=0.0, std=std, generator=generator)
    if drawn != list(full_shape):
        pad = list(full_shape)
        pad[valid[0]] = full_shape[valid[0]] - drawn[valid[0]]
        full = torch.cat([full, full.new_zeros(pad)], dim=valid[0])
    with torch.no_grad():
        param.copy_(shard_tensor(full, shard_dim, parts, tp_rank, tp_size).to(param.dtype))


def shard_tensor(full: torch.Tensor, shard_dim: Optional[int], parts: int, tp_rank: int, tp_size: int) -> torch.Tensor:
    """Slice of ``full`` owned by ``tp_rank``; with ``parts`` > 1 every fused part is sharded separately."""
    if shard_dim is None or tp_size == 1:
        return full
    chunks = _split_parts(full, parts, shard_dim)
    mine = [c.chunk(tp_size, dim=shard_dim)[tp_rank] for c in chunks]
    return torch.cat(mine, dim=shard_dim).contiguous()


def _split_parts(t: torch.Tensor, parts, dim: int):
    """``parts``: number of equal fused parts, or the list of their sizes along ``dim``."""
    if isinstance(parts, int):
        return t.chunk(parts, dim=dim)
    return t.split(list(parts), dim=dim)


def unshard_tensors(shards, shard_dim: Optional[int], parts: int) -> torch.Tensor:
    """Inverse of :func:`shard_tensor` given every rank's shard in rank order."""
    if shard_dim is None or len(shards) == 1:
        return shards[0]
    n = len(shards)
    local_parts = parts if isinstance(parts, int) else [p // n for p in parts]
    per_rank_parts = [_split_parts(s, local_parts, shard_dim) for s in shards]
    nparts = len(per_rank_parts[0])
    merged = [torch.cat([per_rank_parts[r][p] for r in range(n)], dim=shard_dim) for p in range(nparts)]
    return torch.cat(merged, dim=shard_dim).contiguous()
