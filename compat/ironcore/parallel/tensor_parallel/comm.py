"""The reference's autograd communication functions over the tensor-parallel group
(ironcore/parallel/tensor_parallel/comm.py:158-245), mapped onto ``ironcore_b200.parallel.collectives``:

  copy_inputs_to_model_parallel_workers      identity forward, all-reduce backward   (copy_to_tp)
  reduce_inputs_from_model_parallel_workers  all-reduce forward, identity backward   (reduce_from_tp)
  scatter_input_to_model_parallel_workers    keep this rank's slice of the last dim  (scatter_last_dim)
  gather_from_model_parallel_workers(x, a)   gather a sharded tensor; ``a`` is the module that owns it
                                             (``column_parallel`` / ``row_parallel`` / ``concatenated_weights``)
  split_to_model_parallel_workers(x, a)      the inverse: this rank's shard of a full tensor
"""

from ironcore_b200.parallel import collectives as _C
from ironcore_b200.parallel import mesh as _mesh
from ironcore_b200.parallel.tensor_parallel import shard_tensor as _shard, unshard_tensors as _unshard


def _group():
    return _mesh.get_tensor_model_parallel_group()


def copy_inputs_to_model_parallel_workers(x):
    return _C.copy_to_tp(x, _group())


def reduce_inputs_from_model_parallel_workers(x):
    return _C.reduce_from_tp(x, _group())


def scatter_input_to_model_parallel_workers(x):
    return _C.scatter_last_dim(x, _group())


def _layout(attrib):
    parts = getattr(attrib, "concatenated_weights", 1) or 1
    if getattr(attrib, "column_parallel", False):
        return -1, parts
    if getattr(attrib, "row_parallel", False):
        return 0, 1
    return None, 1


def gather_from_model_parallel_workers(x, attrib):
    import torch
    import torch.distributed as dist

    dim, parts = _layout(attrib)
    n = _mesh.get_tensor_model_parallel_world_size()
    if dim is None or n == 1:
        return x
    dim = dim % x.dim()
    shards = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(shards, x.contiguous(), group=_group())
    return _unshard(shards, dim, parts)


def split_to_model_parallel_workers(x, attrib):
    dim, parts = _layout(attrib)
    n = _mesh.get_tensor_model_parallel_world_size()
    if dim is None or n == 1:
        return x
    return _shard(x, dim % x.dim(), parts, _mesh.get_tensor_model_parallel_rank(), n)
