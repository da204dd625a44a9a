"""Symmetric-memory workspaces for the fused compute+collective kernels.

A workspace is one allocation of PyTorch's symmetric-memory allocator, made by every rank of
a process group with the same size and exchanged with ``rendezvous``; afterwards each rank
knows the device address of every peer's copy (NVLink peer pointers through NVSwitch). The
kernels read / write those addresses directly (plain P2P loads and stores, ``multimem`` stores and
reductions through the NVSwitch multicast mapping, release/acquire flags); no TMA multicast and no
library kernel ever sees a peer pointer.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist


@dataclass
class CommPolicy:
    """Process-wide choices for the in-kernel collectives, set from ``config.parallel`` by the trainer.

    nvls: "auto" | "on" | "off". Whether kernels use the NVSwitch multicast mapping (``multimem.st`` /
    ``multimem.ld_reduce``) where the fabric offers one. "auto": broadcast-type transfers (all-gather push,
    parameter broadcast) from 4 ranks up (one store instead of world-1: measured 13 % faster at 4 ranks,
    slower at 2); reduce-type transfers of the tensor-parallel GEMMs stay on P2P stores, which overlap the
    transfer with the remaining tiles (pulling sums through the switch after the last tile measured slower
    at 2 and 4 ranks)."""

    nvls: str = "auto"
    fused_zero: bool = True
    fused_moe: bool = True
    fused_norm_gather: str = "auto"


POLICY = CommPolicy()


def configure(parallel_config) -> CommPolicy:
    for name in ("nvls", "fused_zero", "fused_moe", "fused_norm_gather"):
        if hasattr(parallel_config, name):
            setattr(POLICY, name, getattr(parallel_config, name))
    return POLICY


def nvls_requested(world: int, op: str) -> bool:
    """``op``: "ag" (broadcast-type) or "rs" (reduce-type); see :class:`CommPolicy`."""
    v = str(POLICY.nvls).lower()
    if v in ("0", "false", "off"):
        return False
    if v in ("1", "true", "on"):
        return True
    return op == "ag" and world >= 4


def symmetric_memory_available() -> bool:
    if not (torch.cuda.is_available() and dist.is_initialized()):
        return False
    try:
        import torch.distributed._symmetric_memory as _sm  # noqa: F401

        return True
    except Exception:
        return False


class SymmetricBuffer:
    """``nbytes`` of zero-initialised symmetric memory over ``group``."""

    def __init__(self, nbytes: int, group):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        nbytes = (nbytes + 255) // 256 * 256
        self.nbytes = nbytes
        dev = torch.device("cuda", torch.cuda.current_device())
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.handle = symm_mem.rendezvous(self.local, group)
        self.local.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        if self.peer_ptrs[self.rank] != self.local.data_ptr():
            raise RuntimeError("symmetric memory: local pointer does not match the rendezvous table")
        # Multicast (NVLS) mapping of the same allocation: a store to it lands in every rank's copy, a
        # multimem.ld_reduce returns the sum over the copies. 0 when the fabric has no multicast support.
        try:
            self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        except Exception:
            self.multicast_ptr = 0

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nb].view(dtype).view(*shape)

    def peer_table(self, offset: int) -> torch.Tensor:
        """int64 device tensor [world] with every rank's address of the region at ``offset``."""
        return torch.tensor([p + offset for p in self.peer_ptrs], dtype=torch.int64, device=self.local.device)
