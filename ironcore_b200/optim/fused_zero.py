"""ZeRO-1 optimizer step with its collectives inside the kernels (``csrc/zero_step.cu``).

The flat fp32 gradient buffer and the flat 16-bit parameter buffer of a data-parallel group live in
one symmetric-memory allocation, so the kernels address every peer's copy over NVLink:
``zero_reduce_kernel`` sums this rank's shard of the gradient over all ranks (P2P loads or one
``multimem.ld_reduce`` through the NVSwitch) and publishes its part of the gradient norm;
``zero_adam_kernel`` applies the clip coefficient and Adam to the shard and stores the new parameters
into every rank's buffer (P2P stores or one ``multimem.st``), then waits until all ranks did.
The NCCL composition in :mod:`ironcore_b200.optim.distributed` (reduce-scatter, all-reduce of the
norm, Adam kernel, all-gather) is the fallback and the oracle.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.native import call, dtype_code, ptr, stream_ptr

P, I, L, F = native.P, native.I, native.L, native.F
native.register("icb_zero_step", [I, I, I, I, P, P, P, P, P, P, P, P, P, P, L, P, P, P, P, P, P, P, P,
                                  F, F, F, F, F, F, F, I, P, P])

_CTR_BYTES = 256
_NORM_BYTES = 256


class FusedZeroStep:
    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ready = False
        self.buf = None

    @staticmethod
    def create(group) -> Optional["FusedZeroStep"]:
        from ..parallel.symmetric import POLICY, symmetric_memory_available

        if not POLICY.fused_zero:
            return None
        if not symmetric_memory_available() or dist.get_world_size(group) > 16:
            return None
        return FusedZeroStep(group)

    # called by FlatGroup: returns (param_buf, grad_buf) views of one symmetric allocation
    def allocate(self, flat_group, param_dtype, grad_dtype):
        from ..parallel.symmetric import SymmetricBuffer

        total = flat_group.total
        pbytes = (total * torch.empty((), dtype=param_dtype).element_size() + 255) // 256 * 256
        gbytes = (total * 4 + 255) // 256 * 256
        self._p_off, self._g_off = 0, pbytes
        self._ctr_off = pbytes + gbytes
        self._norm_off = self._ctr_off + _CTR_BYTES
        self.buf = SymmetricBuffer(self._norm_off + _NORM_BYTES, self.group)
        b = self.buf
        self.param_buf = b.view(self._p_off, (total,), param_dtype)
        self.grad_buf = b.view(self._g_off, (total,), torch.float32)
        self.p_dtype = param_dtype
        dev = b.local.device
        self.peer_params = b.peer_table(self._p_off)
        self.peer_grads = b.peer_table(self._g_off)
        self.peer_ctr = b.peer_table(self._ctr_off)
        self.peer_norm = b.peer_table(self._norm_off)
        self.ctr = b.view(self._ctr_off, (4,), torch.int32)
        self.norm_slots = b.view(self._norm_off, (32,), torch.float32)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.scratch = torch.zeros(2, dtype=torch.int32, device=dev)
        self.norm_out = torch.zeros(1, dtype=torch.float32, device=dev)
        self.coef_out = torch.ones(1, dtype=torch.float32, device=dev)
        from ..parallel.symmetric import nvls_requested

        use_mc = b.multicast_ptr != 0 and nvls_requested(self.world, "ag")
        flag = torch.tensor([1 if use_mc else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        self.nvls = bool(int(flag.item()))
        self.ready = True
        return self.param_buf, self.grad_buf

    def step(self, regions, lo, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, step_size, grad_scale, clip,
             master=None):
        n = len(regions)
        arr = (C.c_double * (5 * max(n, 1)))()
        for i, reg in enumerate(regions):
            for j in range(5):
                arr[i * 5 + j] = float(reg[j])
        b = self.buf
        mc = b.multicast_ptr if self.nvls else 0
        call("icb_zero_step", 3, self.rank, self.world, n, C.cast(arr, C.c_void_p), ptr(self.peer_grads),
             (mc + self._g_off) if mc else None, ptr(self.grad_buf), ptr(self.peer_params),
             (mc + self._p_off) if mc else None, ptr(self.param_buf), ptr(master), ptr(exp_avg), ptr(exp_avg_sq),
             int(lo), ptr(self.peer_ctr), ptr(self.ctr), ptr(self.peer_norm), ptr(self.norm_slots),
             ptr(self.epoch_dev), ptr(self.scratch), ptr(self.norm_out), ptr(self.coef_out), float(lr), float(beta1),
             float(beta2), float(eps), float(step_size), float(grad_scale), float(clip), dtype_code(self.p_dtype),
             ptr(native.status_tensor(self.grad_buf.device)), stream_ptr())
        self.epoch_dev.add_(1)
        return self.norm_out.clone()
