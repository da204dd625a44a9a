"""Fused compute+collective paths of tensor parallelism with sequence parallelism.

``FusedTP`` owns two symmetric-memory workspaces shared by every layer of a model:

* gather workspace  : two (call-parity) gathered activation buffers ``[M, d]`` plus the
  per-128-row arrival counters that the peers bump when their pushed shard chunks have
  landed, used by ``icb_ag_gemm`` (all-gather -> GEMM in one kernel);
* scatter workspace : two receive buffers ``[t][M/t][d]`` plus per-tile arrival counters used
  by ``icb_gemm_rs`` (GEMM -> reduce-scatter in one kernel).

Forward and backward of the column- / row-parallel linears map onto these two kernels:

  column fwd  : AG(x) -> GEMM                      (icb_ag_gemm, a_major 0)
  column dgrad: GEMM(dy, W^T) -> RS                (icb_gemm_rs)
  column wgrad: AG(x)^T GEMM dy                    (icb_ag_gemm, a_major 1, accumulates into main_grad)
  row fwd     : GEMM -> RS (+bias +residual)       (icb_gemm_rs)
  row dgrad   : AG(dy) -> GEMM                     (icb_ag_gemm, a_major 0)
  row wgrad   : x^T GEMM gathered(dy)              (plain GEMM on the buffer the dgrad call filled)

Every rank must issue the same sequence of calls (SPMD). Each workspace counts its calls in a
device word that the kernels read as the epoch of their cumulative flags, so a captured CUDA
graph replays correctly; the host-side counter only selects the buffer parity, which is why a
captured region must contain an even number of calls per workspace (checked by the trainer). The ``torch.distributed``
path in :mod:`ironcore_b200.parallel.tensor_parallel` is the fallback and the oracle.
"""

from __future__ import annotations

from typing import Optional

import os

import torch
import torch.distributed as dist

from ..ops import kernels, native
from ..ops.native import call, dtype_code, ptr, stream_ptr
from .symmetric import SymmetricBuffer, symmetric_memory_available

P, I, L = native.P, native.I, native.L
native.register("icb_ag_gemm", [P, P, P, P, P, I, I, I, I, P, P, P, P, P, I, L, L, L, I, I, I, I, P, P, P])
native.register("icb_gemm_rs", [P, P, P, P, P, I, I, I, L, L, L, L, I, I, P, P, P, P, I, I, P, P, P, P])


def _nvls_requested(world: int, op: str) -> bool:
    """Whether ``op`` ("ag" or "rs") uses the NVSwitch multicast form. ``ICB_NVLS=1`` / ``0`` forces it on /
    off for both. By default the all-gather push uses it from 4 ranks up (one multimem.st instead of world-1
    P2P stores: measured 13 % faster at 4 ranks, slower at 2), and the reduce-scatter stays on P2P stores:
    pushing partial tiles while the tensor core still works overlaps better than pulling the sums through
    the switch after the last tile (measured at 2 and 4 ranks)."""
    v = os.environ.get("ICB_NVLS", "auto").lower()
    if v in ("0", "false", "off"):
        return False
    if v in ("1", "true", "on"):
        return True
    return op == "ag" and world >= 4


class FusedTP:
    def __init__(self, tokens: int, width: int, group, dtype=torch.bfloat16, nvls: Optional[bool] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.tokens, self.width, self.dtype = tokens, width, dtype
        if tokens % self.world or (tokens // self.world) % 128 or width % 32:
            raise ValueError("fused TP needs tokens/world to be a multiple of 128 and width a multiple of 32")
        self.rows = tokens // self.world
        es = 2
        self.max_n_tiles = (width + 255) // 256
        # ---- gather workspace ----
        g_data = tokens * width * es
        self._g_off = [0, g_data]
        self._g_ready_off = 2 * g_data
        self._g_signal_off = self._g_ready_off + (tokens // 128) * 4
        g_total = self._g_signal_off + self.world * 4
        self.gbuf = SymmetricBuffer(g_total, group)
        self.g_views = [self.gbuf.view(self._g_off[p], (tokens, width), dtype) for p in range(2)]
        self.g_peers = [self.gbuf.peer_table(self._g_off[p]) for p in range(2)]
        self.g_peer_signal = self.gbuf.peer_table(self._g_signal_off)
        self.g_peer_ready = self.gbuf.peer_table(self._g_ready_off)
        self.g_ready = self.gbuf.view(self._g_ready_off, (tokens // 128,), torch.int32)
        self.g_signal = self.gbuf.view(self._g_signal_off, (self.world,), torch.int32)
        self.g_epoch = 0
        self.g_epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.gbuf.local.device)
        self.last_gathered: Optional[torch.Tensor] = None
        # ---- scatter workspace ----
        r_data = tokens * width * es
        self._r_off = [0, r_data]
        self._r_flags_off = 2 * r_data
        n_flags = (self.rows // 128) * self.max_n_tiles
        r_total = self._r_flags_off + n_flags * 4
        self.rbuf = SymmetricBuffer(r_total, group)
        self.r_peers = [self.rbuf.peer_table(self._r_off[p]) for p in range(2)]
        self.r_peer_flags = self.rbuf.peer_table(self._r_flags_off)
        self.r_flags = self.rbuf.view(self._r_flags_off, (n_flags,), torch.int32)
        self.r_epoch = 0
        self.r_epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.rbuf.local.device)
        # True: forward keeps the gathered activations (32 MiB at 4096 x 4096) for the weight gradient;
        # False: backward re-gathers inside the wgrad kernel (less memory, exposed transfer).
        self.save_gathered = True
        # NVLS: push the gathered shard once with multimem.st and reduce the scattered partials with
        # multimem.ld_reduce when the symmetric allocations have a multicast mapping on every rank.
        have = torch.tensor([1 if (self.gbuf.multicast_ptr and self.rbuf.multicast_ptr) else 0],
                            dtype=torch.int32, device=self.gbuf.local.device)
        if self.world > 1:
            dist.all_reduce(have, op=dist.ReduceOp.MIN, group=group)
        have = self.world > 1 and int(have.item()) == 1
        self.nvls_ag = bool(have and (_nvls_requested(self.world, "ag") if nvls is None else nvls))
        self.nvls_rs = bool(have and (_nvls_requested(self.world, "rs") if nvls is None else nvls))
        self.nvls = self.nvls_ag or self.nvls_rs

    # ------------------------------------------------------------------ raw kernels
    def ag_gemm(self, x_shard: torch.Tensor, b: torch.Tensor, *, a_major: int, b_major: int, n: int,
                bias=None, out=None, residual=None, out_dtype=None) -> torch.Tensor:
        """AG(x_shard) (x) b. a_major 0: [tokens, width] @ b -> [tokens, n];
        a_major 1: gathered^T @ b[tokens, n] -> [width, n]."""
        if x_shard.shape != (self.rows, self.width) or x_shard.dtype != self.dtype:
            raise ValueError(f"fused gather expects a [{self.rows}, {self.width}] {self.dtype} shard")
        self.g_epoch += 1
        par = self.g_epoch & 1
        gathered = self.g_views[par]
        gathered[self.rank * self.rows:(self.rank + 1) * self.rows].copy_(x_shard)
        m = self.tokens if a_major == 0 else self.width
        out_dtype = out_dtype or (out.dtype if out is not None else self.dtype)
        if out is None:
            out = torch.empty((m, n), dtype=out_dtype, device=x_shard.device)
        ldr = residual.stride(0) if residual is not None else 0
        call("icb_ag_gemm", ptr(gathered), ptr(self.g_peers[par]), ptr(self.g_peer_ready), ptr(self.g_signal),
             ptr(self.g_ready), self.rank, self.world, self.rows, self.width, ptr(self.g_epoch_dev), ptr(b), ptr(out),
             ptr(bias), ptr(residual), int(n), b.stride(0), out.stride(0), ldr, int(a_major), int(b_major),
             dtype_code(self.dtype), 1 if out_dtype == torch.float32 else 0,
             ptr(native.status_tensor(x_shard.device)), stream_ptr(),
             (self.gbuf.multicast_ptr + self._g_off[par]) if self.nvls_ag else None)
        self.g_epoch_dev.add_(1)
        self.last_gathered = gathered
        return out

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, *, b_major: int, bias=None, residual=None) -> torch.Tensor:
        """reduce_scatter_rows(a[tokens, k] (x) b) -> [tokens / world, width]."""
        if a.shape[0] != self.tokens or a.dtype != self.dtype:
            raise ValueError("fused reduce-scatter expects the full token dimension")
        n = self.width
        k = a.shape[1]
        self.r_epoch += 1
        par = self.r_epoch & 1
        out = torch.empty((self.rows, n), dtype=self.dtype, device=a.device)
        ldr = residual.stride(0) if residual is not None else 0
        recv_ptr = self.rbuf.local.data_ptr() + self._r_off[par]
        call("icb_gemm_rs", ptr(a), ptr(b), ptr(out), ptr(bias), ptr(residual), self.tokens, n, k, a.stride(0),
             b.stride(0), out.stride(0), ldr, int(b_major), dtype_code(self.dtype), ptr(self.r_peers[par]),
             ptr(self.r_peer_flags), recv_ptr, ptr(self.r_flags), self.rank, self.world, ptr(self.r_epoch_dev),
             ptr(native.status_tensor(a.device)), stream_ptr(),
             (self.rbuf.multicast_ptr + self._r_off[par]) if self.nvls_rs else None)
        self.r_epoch_dev.add_(1)
        return out

    # ------------------------------------------------------------------ autograd entry points
    def allgather_linear(self, x_shard, weight, bias=None):
        return _AllGatherLinear.apply(x_shard, weight, bias, self)

    def linear_reduce_scatter(self, x, weight, bias=None, residual=None):
        return _LinearReduceScatter.apply(x, weight, bias, residual, self)

    def supports(self, x: torch.Tensor) -> bool:
        return x.dtype == self.dtype and x.is_cuda


def _accumulate_or_return(weight, compute):
    """Weight gradient: add into the flat fp32/16-bit main_grad buffer when the optimizer
    engine installed one (returns None for autograd), else return a fresh tensor."""
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        compute(main_grad)
        weight.grad_ready = True
        return None
    return compute(None)


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, bias, ws: FusedTP):
        x2 = x_shard.reshape(-1, x_shard.shape[-1]).contiguous()
        y = ws.ag_gemm(x2, weight, a_major=0, b_major=1, n=weight.shape[1], bias=bias)
        # Keep the gathered activations for the weight gradient (the workspace buffer is reused two
        # calls later). A re-gather inside the wgrad kernel cannot hide its transfer: the reduction
        # runs over the gathered rows, so every output tile needs all of them at once.
        x_full = ws.last_gathered.clone() if ws.save_gathered else x2
        ctx.save_for_backward(x_full, weight)
        ctx.ws = ws
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        ws: FusedTP = ctx.ws
        dy = dy.contiguous()
        dx = ws.gemm_rs(dy, weight, b_major=0) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            n = weight.shape[1]

            def compute(acc):
                if ws.save_gathered:
                    if acc is not None:
                        return kernels.mm_tn(x2, dy, out=acc, residual=acc, out_dtype=acc.dtype)
                    return kernels.mm_tn(x2, dy)
                if acc is not None:
                    return ws.ag_gemm(x2, dy, a_major=1, b_major=1, n=n, out=acc, residual=acc, out_dtype=acc.dtype)
                return ws.ag_gemm(x2, dy, a_major=1, b_major=1, n=n)

            dw = _accumulate_or_return(weight, compute)
        db = dy.sum(0, dtype=torch.float32).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, ws: FusedTP):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        res2 = residual.reshape(-1, weight.shape[1]).contiguous() if residual is not None else None
        y = ws.gemm_rs(x2, weight, b_major=1, bias=bias, residual=res2)
        ctx.save_for_backward(x2, weight)
        ctx.ws = ws
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x2, weight = ctx.saved_tensors
        ws: FusedTP = ctx.ws
        dy_shard = dy_shard.contiguous()
        # dX_local = AG(dy) @ W^T ; the gathered dy stays in the workspace for the weight gradient
        dx = ws.ag_gemm(dy_shard, weight, a_major=0, b_major=0, n=weight.shape[0])
        dy_full = ws.last_gathered
        dw = None
        if ctx.needs_input_grad[1]:
            def compute(acc):
                if acc is not None:
                    return kernels.mm_tn(x2, dy_full, out=acc, residual=acc, out_dtype=acc.dtype)
                return kernels.mm_tn(x2, dy_full)

            dw = _accumulate_or_return(weight, compute)
        db = dy_shard.sum(0, dtype=torch.float32).to(dy_shard.dtype) if ctx.has_bias and ctx.needs_input_grad[2] \
            else None
        dres = dy_shard if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, None


def attach_fused_tp(model, config) -> Optional[FusedTP]:
    """Create the shared workspaces and hand them to every sequence-parallel column / row
    parallel linear of ``model``. Returns None (and leaves the NCCL path active) when
    symmetric memory is unavailable or the shapes do not fit the kernels' tiling."""
    from . import mesh
    from .tensor_parallel import ColumnParallelLinear, RowParallelLinear

    if not symmetric_memory_available():
        return None
    group = mesh.get_tensor_model_parallel_group()
    t = mesh.get_tensor_model_parallel_world_size()
    tokens = config.trainer.micro_batch_size * config.model.max_seq_len
    width = config.model.d_model
    if t < 2 or tokens % t or (tokens // t) % 128 or width % 32:
        return None
    from ..models.language_model import get_model_dtype

    dtype = get_model_dtype(config)
    if dtype not in (torch.bfloat16, torch.float16):
        return None
    ws = FusedTP(tokens, width, group, dtype)
    head = getattr(model, "output_layer", None)
    for mod in model.modules():
        if mod is head:
            continue   # keeps the number of fused calls per micro-batch even (needed for CUDA-graph replay)
        if isinstance(mod, ColumnParallelLinear) and mod.sequence_parallel and mod.in_features == width:
            mod.fused = ws
        elif isinstance(mod, RowParallelLinear) and mod.sequence_parallel and mod.out_features == width:
            mod.fused = ws
    return ws
