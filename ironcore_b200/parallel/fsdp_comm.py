"""FSDP collectives as kernels over symmetric memory (``csrc/fsdp_comm.cu``); opt-in building block.

``FsdpCommPool`` owns one symmetric allocation per data-parallel group with ``slots`` full-parameter
buffers and ``slots`` flat-gradient buffers of the largest unit, plus the counters of the two kernels:

  gather(shard, slot)                  -> view of the slot's full buffer, complete when the kernel is
  reduce_scatter(slot, grad_shard, s)  -> grad_shard += s * sum over ranks of the slot's flat gradient range

Both run on the current stream, so a caller overlaps them with compute by issuing them on a side stream.
The parameter gather writes with P2P stores (or one ``multimem.st`` when the fabric offers multicast), the
reduce-scatter reads its range from every rank (or one ``multimem.ld_reduce``) and fuses the cast, the
scale and the accumulation into the fp32 gradient shard. The NCCL calls in
:mod:`ironcore_b200.parallel.fsdp` are the default path and the oracle.
"""

from __future__ import annotations


import torch
import torch.distributed as dist

from ..ops import native
from ..ops.native import call, dtype_code, ptr, stream_ptr
from .symmetric import SymmetricBuffer

P, I, L, F = native.P, native.I, native.L, native.F
native.register("icb_fsdp_gather", [P, L, P, P, I, I, P, P, P, P, P, P])
native.register("icb_fsdp_reduce_scatter", [P, P, P, L, F, I, I, I, P, P, P, P, P, P])


class FsdpCommPool:
    def __init__(self, group, max_unit_elems: int, param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                 slots: int = 2, flat_slots=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if max_unit_elems % (8 * self.world):
            raise ValueError("unit size must be a multiple of 8 * world elements")
        self.max_elems, self.slots = max_unit_elems, slots
        self.param_dtype, self.reduce_dtype = param_dtype, reduce_dtype
        pes = torch.empty((), dtype=param_dtype).element_size()
        res = torch.empty((), dtype=reduce_dtype).element_size()
        self._full_bytes = (max_unit_elems * pes + 255) // 256 * 256
        self._flat_bytes = (max_unit_elems * res + 255) // 256 * 256
        flat_slots = slots if flat_slots is None else flat_slots     # 0: gather only, no gradient buffers
        self.flat_slots = flat_slots
        self._flat_off = slots * self._full_bytes
        self._ctr_off = self._flat_off + flat_slots * self._flat_bytes
        self.buf = SymmetricBuffer(self._ctr_off + 256, group)
        dev = self.buf.local.device
        self.ctr = self.buf.view(self._ctr_off, (4,), torch.int32)
        self.peer_ctr = self.buf.peer_table(self._ctr_off)
        self.peer_full = [self.buf.peer_table(s * self._full_bytes) for s in range(slots)]
        self.peer_flat = [self.buf.peer_table(self._flat_off + s * self._flat_bytes) for s in range(flat_slots)]
        self.gather_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.reduce_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(2, dtype=torch.int32, device=dev)
        from .symmetric import nvls_requested

        use_mc = self.buf.multicast_ptr != 0 and nvls_requested(self.world, "ag")
        flag = torch.tensor([1 if use_mc else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        self.nvls = bool(int(flag.item()))

    def full_view(self, slot: int, elems: int) -> torch.Tensor:
        return self.buf.view(slot * self._full_bytes, (elems,), self.param_dtype)

    def flat_view(self, slot: int, elems: int) -> torch.Tensor:
        return self.buf.view(self._flat_off + slot * self._flat_bytes, (elems,), self.reduce_dtype)

    def gather(self, shard: torch.Tensor, slot: int) -> torch.Tensor:
        """All-gather ``shard`` (every rank's has the same length) into the slot's full buffer."""
        n = shard.numel()
        if n % 8 or n * self.world > self.max_elems or shard.dtype != self.param_dtype:
            raise ValueError("shard does not fit the pool")
        mc = (self.buf.multicast_ptr + slot * self._full_bytes) if self.nvls else None
        call("icb_fsdp_gather", ptr(shard), n, ptr(self.peer_full[slot]), mc, self.rank, self.world, ptr(self.peer_ctr),
             ptr(self.ctr), ptr(self.gather_epoch), ptr(self.ticket), ptr(native.status_tensor(shard.device)),
             stream_ptr())
        self.gather_epoch.add_(1)
        return self.full_view(slot, n * self.world)

    def reduce_scatter(self, slot: int, grad_shard: torch.Tensor, scale: float = 1.0) -> None:
        """grad_shard (fp32) += scale * sum over ranks of this rank's range of the slot's flat gradient."""
        n = grad_shard.numel()
        if n % 8 or n * self.world > self.max_elems or grad_shard.dtype != torch.float32:
            raise ValueError("gradient shard does not fit the pool")
        mc = (self.buf.multicast_ptr + self._flat_off + slot * self._flat_bytes) if self.nvls else None
        call("icb_fsdp_reduce_scatter", ptr(self.peer_flat[slot]), mc, ptr(grad_shard), n, float(scale),
             dtype_code(self.reduce_dtype), self.rank, self.world, ptr(self.peer_ctr), ptr(self.ctr),
             ptr(self.reduce_epoch), ptr(self.ticket[1:]), ptr(native.status_tensor(grad_shard.device)), stream_ptr())
        self.reduce_epoch.add_(1)
