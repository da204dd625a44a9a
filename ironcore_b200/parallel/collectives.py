"""Autograd-aware collectives for tensor / sequence / expert parallelism over
``torch.distributed`` (NCCL on GPU, Gloo on CPU). These are the baseline data plane
and the oracle for the fused compute+collective kernels.

Conjugate pairs (forward / backward):
  copy_to_tp            identity            / all-reduce
  reduce_from_tp        all-reduce          / identity
  gather_from_sp        all-gather (dim 0)  / reduce-scatter (dim 0)
  reduce_scatter_to_sp  reduce-scatter      / all-gather
  scatter_to_sp         keep own dim-0 chunk/ all-gather
  gather_last_dim       all-gather (dim -1) / keep own chunk
  all_to_all            all-to-all (splits) / all-to-all (transposed splits)
(Behavioural reference: ironcore/parallel/tensor_parallel/comm.py:24-223; the
sequence-parallel and all-to-all forms have no counterpart there.)
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def _rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


# ----------------------------------------------------------------- raw helpers (no autograd)
def all_reduce_(t: torch.Tensor, group, op=None) -> torch.Tensor:
    if _size(group) > 1:
        dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group)
    return t


def all_gather_dim0(t: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return t
    t = t.contiguous()
    out = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t, group=group)
    return out


def reduce_scatter_dim0(t: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return t
    t = t.contiguous()
    if t.shape[0] % n != 0:
        raise ValueError(f"dim 0 ({t.shape[0]}) not divisible by group size {n}")
    out = torch.empty((t.shape[0] // n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if t.device.type == "cpu":
        # Gloo has no reduce_scatter: all-reduce then keep the local chunk.
        tmp = t.clone()
        dist.all_reduce(tmp, group=group)
        out.copy_(tmp.chunk(n, dim=0)[_rank(group)])
    else:
        dist.reduce_scatter_tensor(out, t, group=group)
    return out


def all_gather_last_dim(t: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


def split_last_dim(t: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return t
    return t.chunk(n, dim=-1)[_rank(group)].contiguous()


def split_dim0(t: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return t
    return t.chunk(n, dim=0)[_rank(group)].contiguous()


def all_to_all_single(t: torch.Tensor, out_splits: Optional[List[int]], in_splits: Optional[List[int]], group):
    n = _size(group)
    if n == 1:
        return t
    t = t.contiguous()
    rows = sum(out_splits) if out_splits is not None else t.shape[0]
    out = torch.empty((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if t.device.type == "cpu":
        # Gloo has no all_to_all: exchange the per-peer slices with isend / irecv.
        ins = in_splits if in_splits is not None else [t.shape[0] // n] * n
        outs = out_splits if out_splits is not None else [rows // n] * n
        send = list(t.split(ins, dim=0))
        recv = [torch.empty((outs[i],) + tuple(t.shape[1:]), dtype=t.dtype) for i in range(n)]
        _gloo_all_to_all(recv, send, group)
        out = torch.cat(recv, dim=0)
    else:
        dist.all_to_all_single(out, t, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    return out


def _gloo_all_to_all(recv, send, group):
    n, me = _size(group), _rank(group)
    ranks = dist.get_process_group_ranks(group)
    reqs = []
    for i in range(n):
        if i == me:
            recv[i].copy_(send[i])
            continue
        reqs.append(dist.isend(send[i].contiguous(), dst=ranks[i], group=group))
        reqs.append(dist.irecv(recv[i], src=ranks[i], group=group))
    for r in reqs:
        r.wait()


# ----------------------------------------------------------------- autograd functions
class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_(g.contiguous().clone(), ctx.group), None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_(x.contiguous().clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_dim0(g, ctx.group), None


class _ReduceScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group), None


class _ScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return split_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group), None


class _GatherToFull(torch.autograd.Function):
    """all-gather dim 0 forward, keep own chunk backward (used where every rank then does
    the same replicated computation, e.g. gathering SP shards before the LM head loss)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return split_dim0(g, ctx.group), None


class _GatherLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_last_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        return split_last_dim(g, ctx.group), None


class _ScatterLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return split_last_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_last_dim(g, ctx.group), None


class _AllReduceSum(torch.autograd.Function):
    """Sum over the group in forward, identity in backward (each rank's contribution has
    gradient 1 with respect to the replicated result)."""

    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_(x.contiguous().clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        return all_to_all_single(x, out_splits, in_splits, group)

    @staticmethod
    def backward(ctx, g):
        return all_to_all_single(g, ctx.in_splits, ctx.out_splits, ctx.group), None, None, None


def copy_to_tp(x, group):
    return x if _size(group) == 1 else _CopyToTP.apply(x, group)


def reduce_from_tp(x, group):
    return x if _size(group) == 1 else _ReduceFromTP.apply(x, group)


def gather_from_sp(x, group):
    return x if _size(group) == 1 else _GatherFromSP.apply(x, group)


def reduce_scatter_to_sp(x, group):
    return x if _size(group) == 1 else _ReduceScatterToSP.apply(x, group)


def scatter_to_sp(x, group):
    return x if _size(group) == 1 else _ScatterToSP.apply(x, group)


def gather_to_full(x, group):
    return x if _size(group) == 1 else _GatherToFull.apply(x, group)


def gather_last_dim(x, group):
    return x if _size(group) == 1 else _GatherLastDim.apply(x, group)


def scatter_last_dim(x, group):
    return x if _size(group) == 1 else _ScatterLastDim.apply(x, group)


def all_reduce_sum(x, group):
    return x if _size(group) == 1 else _AllReduceSum.apply(x, group)


def all_to_all(x, out_splits, in_splits, group):
    return x if _size(group) == 1 else _AllToAll.apply(x, out_splits, in_splits, group)


# reference-compatible aliases (ironcore/parallel/tensor_parallel/comm.py)
copy_inputs_to_model_parallel_workers = copy_to_tp
reduce_from_model_parallel_workers = reduce_from_tp
scatter_to_model_parallel_workers = scatter_last_dim
gather_from_model_parallel_workers = gather_last_dim
