"""Process bootstrap and the TP x DP (x EP) process-group mesh.

One process per GPU. ``torch.distributed`` (NCCL on CUDA, Gloo on CPU) is the control
plane and the baseline data plane; the fused kernels use symmetric memory on top.

Rank layout (tp = 4, world = 16): TP groups are contiguous ranks ``[0..3], [4..7], ...``;
DP groups stride by tp ``[0,4,8,12], [1,5,9,13], ...``; an EP group is a contiguous
block of ``ep`` members of one DP group and the expert-data-parallel group collects
the ranks holding the same expert shard.
(Behavioural reference: ironcore/parallel/parallel.py:24-69,
ironcore/parallel/parallel_states.py:27-150.)
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    tp_size: int = 1
    dp_size: int = 1
    ep_size: int = 1
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    ep_group: Optional[object] = None
    edp_group: Optional[object] = None   # ranks that replicate the same expert shard
    tp_ranks: List[int] = field(default_factory=lambda: [0])
    dp_ranks: List[int] = field(default_factory=lambda: [0])
    ep_ranks: List[int] = field(default_factory=lambda: [0])
    edp_ranks: List[int] = field(default_factory=lambda: [0])
    sequence_parallel: bool = False
    initialized: bool = False

    @property
    def tp_rank(self) -> int:
        return self.tp_ranks.index(self.rank) if self.rank in self.tp_ranks else 0

    @property
    def dp_rank(self) -> int:
        return self.dp_ranks.index(self.rank) if self.rank in self.dp_ranks else 0

    @property
    def ep_rank(self) -> int:
        return self.ep_ranks.index(self.rank) if self.rank in self.ep_ranks else 0


_STATE = ParallelState()


def state() -> ParallelState:
    return _STATE


def mesh_layout(world_size: int, tp: int, ep: int = 1):
    """Pure function: the rank lists of every group. Returns dict of lists of lists."""
    if world_size % tp != 0:
        raise ValueError(f"world size {world_size} not divisible by tensor parallel size {tp}")
    dp = world_size // tp
    if dp % ep != 0:
        raise ValueError(f"data parallel size {dp} not divisible by expert parallel size {ep}")
    tp_groups = [list(range(i * tp, (i + 1) * tp)) for i in range(dp)]
    dp_groups = [list(range(i, world_size, tp)) for i in range(tp)]
    ep_groups, edp_groups = [], []
    for g in dp_groups:
        for j in range(0, dp, ep):
            ep_groups.append(g[j:j + ep])
        for j in range(ep):
            edp_groups.append(g[j::ep])
    return {"tp": tp_groups, "dp": dp_groups, "ep": ep_groups, "edp": edp_groups}


def device_type() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def initialize_process(config) -> None:
    """Select the device and create the default process group (idempotent).
    World size 1 without rendezvous variables runs without a process group."""
    p = config.parallel
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(p.local_rank % max(torch.cuda.device_count(), 1))
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    if config.utils.deterministic:
        torch.backends.cudnn.deterministic = True
    if dist.is_initialized():
        return
    if p.world_size <= 1 and "MASTER_ADDR" not in os.environ:
        return
    backend = "nccl" if use_cuda and p.dist_backend == "nccl" else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    timeout = datetime.timedelta(minutes=float(p.timeout_minute or 10.0))
    kwargs = {}
    if use_cuda and backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=backend, rank=max(p.rank, 0), world_size=p.world_size, timeout=timeout, **kwargs)


def initialize_model_parallel(tensor_model_parallel_size: int = 1, expert_model_parallel_size: int = 1,
                              sequence_parallel: bool = False, timeout_in_minutes: float = 10.0) -> ParallelState:
    """Build the TP / DP / EP / expert-DP groups. Every rank creates every group (a
    ``new_group`` requirement); without a process group this records the trivial mesh."""
    global _STATE
    st = ParallelState(sequence_parallel=sequence_parallel and tensor_model_parallel_size > 1)
    if not dist.is_initialized():
        if tensor_model_parallel_size != 1 or expert_model_parallel_size != 1:
            raise RuntimeError("model parallelism needs an initialised process group")
        st.initialized = True
        _STATE = st
        return st
    world, rank = dist.get_world_size(), dist.get_rank()
    layout = mesh_layout(world, tensor_model_parallel_size, expert_model_parallel_size)
    timeout = datetime.timedelta(minutes=float(timeout_in_minutes))
    st.world_size, st.rank = world, rank
    st.tp_size = tensor_model_parallel_size
    st.dp_size = world // tensor_model_parallel_size
    st.ep_size = expert_model_parallel_size
    for kind in ("tp", "dp", "ep", "edp"):
        for ranks in layout[kind]:
            grp = dist.new_group(ranks=ranks, timeout=timeout)
            if rank in ranks:
                setattr(st, f"{kind}_group", grp)
                setattr(st, f"{kind}_ranks", ranks)
    st.initialized = True
    _STATE = st
    return st


def destroy_model_parallel() -> None:
    global _STATE
    _STATE = ParallelState()


def finalize_process() -> None:
    if dist.is_initialized():
        try:
            dist.barrier()
        finally:
            dist.destroy_process_group()
    destroy_model_parallel()


# ------------------------------------------------------------------ getters (reference-compatible names)
def model_parallel_is_initialized() -> bool:
    return _STATE.initialized


def get_tensor_model_parallel_group():
    return _STATE.tp_group


def get_tensor_model_parallel_world_size() -> int:
    return _STATE.tp_size


def get_tensor_model_parallel_rank() -> int:
    return _STATE.tp_rank


def get_tensor_model_parallel_src_rank() -> int:
    return _STATE.tp_ranks[0]


def get_data_parallel_group():
    return _STATE.dp_group


def get_data_parallel_world_size() -> int:
    return _STATE.dp_size


def get_data_parallel_rank() -> int:
    return _STATE.dp_rank


def get_expert_model_parallel_group():
    return _STATE.ep_group


def get_expert_model_parallel_world_size() -> int:
    return _STATE.ep_size


def get_expert_model_parallel_rank() -> int:
    return _STATE.ep_rank


def get_expert_data_parallel_group():
    return _STATE.edp_group


def sequence_parallel_enabled() -> bool:
    return _STATE.sequence_parallel and _STATE.tp_size > 1


def get_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def is_rank_zero() -> bool:
    return get_rank() == 0


def global_rank_of(group, group_rank: int) -> int:
    """Global rank of ``group_rank`` within ``group`` (the default group maps to itself)."""
    if group is None or not dist.is_initialized() or group is dist.group.WORLD:
        return int(group_rank)
    return int(dist.get_global_rank(group, group_rank))
