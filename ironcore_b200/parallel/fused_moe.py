"""Expert-parallel token exchange inside CUDA kernels (``csrc/moe_comm.cu``).

``FusedEP`` owns one symmetric-memory workspace per expert-parallel group, shared by all MoE
layers: a receive buffer ``[cap, d]`` in the grouped GEMM's layout (rows sorted by local expert,
segments padded to 128 rows), an expert-output buffer ``[cap, d]``, the counts matrix
``[ep, E]`` and four cumulative counters.

  dispatch : ``icb_moe_count`` (histogram, in-run positions, counts published to every rank)
             + ``icb_moe_push`` (destination rows from the counts matrix, rows copied with P2P stores
             into the owners' buffers, GEMM tables written, padding rows zeroed)
  combine  : ``icb_moe_pull`` (each token reads its k expert-output rows from the owners with P2P
             loads, weighted sum in fp32)

The backward passes are the same two kernels with the roles swapped: the gradient of combine pushes
``w * dout`` rows to the recorded destinations, the gradient of dispatch pulls and sums the k rows
of ``d(xp)``. Nothing on this path synchronises with the host. The ``all_to_all`` composition in
:mod:`ironcore_b200.models.moe` is the fallback and the oracle.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.native import call, dtype_code, ptr, stream_ptr
from .symmetric import SymmetricBuffer, symmetric_memory_available

P, I = native.P, native.I
native.register("icb_moe_count", [P, I, I, I, I, P, P, P, P, P, P])
native.register("icb_moe_push", [P, P, P, P, P, I, I, I, I, I, I, I, I, P, P, P, P, P, P, P, P, P, P, P, P, P, P])
native.register("icb_moe_pull", [P, P, P, P, P, P, I, I, I, I, I, I, I, P, P, P, P, P, I, P, P])


class FusedEP:
    def __init__(self, group, num_experts: int, top_k: int, max_tokens: int, d_model: int, dtype, factor: float):
        self.group = group
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E, self.top_k, self.d, self.dtype = num_experts, top_k, d_model, dtype
        self.e_local = num_experts // self.ep
        slots = max_tokens * top_k
        rows = int(min(self.ep, max(1.0, factor)) * slots)
        self.cap = (rows + 127) // 128 * 128 + self.e_local * 128
        self.max_tokens = max_tokens
        es = 2
        data = self.cap * d_model * es
        self._recv_off, self._y_off = 0, data
        self._counts_off = 2 * data
        self._ctr_off = self._counts_off + (self.ep * self.E * 4 + 255) // 256 * 256
        self.buf = SymmetricBuffer(self._ctr_off + 256, group)
        b = self.buf
        dev = b.local.device
        self.recv = b.view(self._recv_off, (self.cap, d_model), dtype)
        self.ybuf = b.view(self._y_off, (self.cap, d_model), dtype)
        self.counts = b.view(self._counts_off, (self.ep, self.E), torch.int32)
        self.ctr = b.view(self._ctr_off, (4,), torch.int32)
        self.peer_recv = b.peer_table(self._recv_off)
        self.peer_y = b.peer_table(self._y_off)
        self.peer_counts = b.peer_table(self._counts_off)
        self.peer_ctr = b.peer_table(self._ctr_off)
        self.hist = torch.zeros(self.E, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(4, dtype=torch.int32, device=dev)
        self.count_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.push_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.pull_epoch = torch.zeros(1, dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------ raw kernels
    def _status(self):
        return ptr(native.status_tensor(self.recv.device))

    def dispatch(self, x: torch.Tensor, expert: torch.Tensor):
        """x [T, d], expert int32 [T * k] -> (xp [cap, d] copy of the receive buffer, dest int32 [T * k],
        seg_offsets int32 [e_local + 1], tile_expert int32 [cap / 128], counts int32 [ep, E])."""
        s = expert.numel()
        if x.shape[0] > self.max_tokens or x.shape[1] != self.d or x.dtype != self.dtype:
            raise ValueError("fused expert dispatch: unexpected activation shape or dtype")
        dev = x.device
        pos = torch.empty(s, dtype=torch.int32, device=dev)
        dest = torch.empty(s, dtype=torch.int32, device=dev)
        seg = torch.empty(self.e_local + 1, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(self.cap // 128, dtype=torch.int32, device=dev)
        counts = torch.empty((self.ep, self.E), dtype=torch.int32, device=dev)
        call("icb_moe_count", ptr(expert), s, self.E, self.ep, self.rank, ptr(self.hist), ptr(pos),
             ptr(self.peer_counts), ptr(self.peer_ctr), ptr(self.ticket), stream_ptr())
        self.count_epoch.add_(1)
        call("icb_moe_push", ptr(x), ptr(expert), ptr(pos), None, ptr(dest), s, self.E, self.ep, self.rank, self.top_k,
             0, self.d, self.cap, ptr(self.peer_recv), ptr(self.recv), ptr(self.counts), None, ptr(self.peer_ctr),
             ptr(self.ctr), ptr(self.count_epoch), ptr(self.push_epoch), ptr(seg), ptr(tile_expert), ptr(counts),
             ptr(self.ticket[1:]), self._status(), stream_ptr())
        self.push_epoch.add_(1)
        return self.recv.clone(), dest, seg, tile_expert, counts

    def push_rows(self, rows: torch.Tensor, expert: torch.Tensor, dest: torch.Tensor, counts: torch.Tensor):
        """rows [T * k, d] go to the recorded destinations; returns a copy of the receive buffer [cap, d]."""
        s = expert.numel()
        call("icb_moe_push", ptr(rows), ptr(expert), None, ptr(dest), None, s, self.E, self.ep, self.rank, self.top_k,
             1, self.d, self.cap, ptr(self.peer_recv), ptr(self.recv), ptr(self.counts), ptr(counts),
             ptr(self.peer_ctr), ptr(self.ctr), ptr(self.count_epoch), ptr(self.push_epoch), None, None, None,
             ptr(self.ticket[1:]), self._status(), stream_ptr())
        self.push_epoch.add_(1)
        return self.recv.clone()

    def pull(self, yp: torch.Tensor, expert: torch.Tensor, dest: torch.Tensor, tokens: int, weight=None, addend=None,
             keep_rows: bool = False):
        """out[t] = addend[t] + sum_k weight[t, k] * yp_owner[dest[t, k]]; yp is this rank's [cap, d] buffer."""
        self.ybuf.copy_(yp)
        out = torch.empty((tokens, self.d), dtype=self.dtype, device=yp.device)
        rows = torch.empty((tokens * self.top_k, self.d), dtype=self.dtype, device=yp.device) if keep_rows else None
        call("icb_moe_pull", ptr(expert), ptr(dest), ptr(weight), ptr(addend), ptr(out), ptr(rows), tokens, self.top_k,
             self.E, self.ep, self.rank, self.d, self.cap, ptr(self.peer_y), ptr(self.peer_ctr), ptr(self.ctr),
             ptr(self.pull_epoch), ptr(self.ticket[2:]), dtype_code(self.dtype), self._status(), stream_ptr())
        self.pull_epoch.add_(1)
        return out, rows


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, expert, ws: FusedEP):
        xp, dest, seg, tile_expert, counts = ws.dispatch(x.contiguous(), expert)
        ctx.save_for_backward(expert, dest)
        ctx.ws, ctx.tokens = ws, x.shape[0]
        ctx.mark_non_differentiable(dest, seg, tile_expert, counts)
        return xp, dest, seg, tile_expert, counts

    @staticmethod
    def backward(ctx, dxp, *_):
        expert, dest = ctx.saved_tensors
        dx, _ = ctx.ws.pull(dxp.contiguous(), expert, dest, ctx.tokens)
        return dx, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, w, expert, dest, counts, ws: FusedEP):
        tokens = w.shape[0]
        wf = w.float().contiguous()
        out, rows = ws.pull(yp.contiguous(), expert, dest, tokens, weight=wf, keep_rows=True)
        ctx.save_for_backward(wf, rows, expert, dest, counts)
        ctx.ws, ctx.w_dtype = ws, w.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        wf, rows, expert, dest, counts = ctx.saved_tensors
        ws: FusedEP = ctx.ws
        t, k = wf.shape
        dout = dout.contiguous()
        dw = torch.einsum("td,tkd->tk", dout.float(), rows.view(t, k, -1).float()).to(ctx.w_dtype)
        drows = (dout.unsqueeze(1).float() * wf.unsqueeze(-1)).to(dout.dtype).view(t * k, -1)
        dyp = ws.push_rows(drows, expert, dest, counts)
        return dyp, dw, None, None, None, None


def fused_dispatch(x, expert, ws: FusedEP):
    return _Dispatch.apply(x, expert, ws)


def fused_combine(yp, w, expert, dest, counts, ws: FusedEP):
    return _Combine.apply(yp, w, expert, dest, counts, ws)


_WORKSPACES = {}
# Largest expert-parallel group the in-kernel exchange is used for. Two ranks pass the numerics tests and full-size
# training runs. A full-size run on four ranks (64 experts, top-6, 8192 tokens per micro-batch, 16 layers) ended
# twice with an illegal memory access in its fourth step. The likeliest chain, found by reading afterwards: the
# receive buffers held 2 x the mean load (the worst case only for 2 ranks), an overflow set the status block, the
# flag waits of later kernels then returned at once, a dispatch that never saw its counts left its tables
# uninitialised, and the backward push derived a negative row from them. Each link is closed now (worst-case
# buffers up to 4 ranks, defined tables when the counts do not arrive, a guard on the row), but none of it has run
# on 4 GPUs since, so larger groups keep taking the all-to-all composition until it has.
MAX_VERIFIED_EP = 2


def get_fused_ep(group, num_experts, top_k, max_tokens, d_model, dtype, factor: float = 0.0) -> Optional[FusedEP]:
    """Shared workspace for all MoE layers with the same geometry; None when the fused path cannot run.

    ``factor``: rows of every receive buffer as a multiple of one rank's slots (tokens x top_k). 0 = dropless up to
    4 ranks (the worst case, every slot of every rank on one owner) and 4 x the mean load beyond, where the worst
    case would multiply the expert activations by the group size; a positive value is a capacity factor. Rows that
    do not fit are dropped (they contribute nothing, forward and backward) and the status block reports it."""
    from .symmetric import POLICY

    if not POLICY.fused_moe:
        return None
    if not symmetric_memory_available() or dtype not in (torch.bfloat16, torch.float16):
        return None
    ep = dist.get_world_size(group)
    if ep < 2 or ep > 16 or num_experts > 256 or d_model % 8:
        return None
    if ep > MAX_VERIFIED_EP:
        return None
    if factor <= 0:
        factor = float(min(ep, 4))
    key = (id(group), num_experts, top_k, max_tokens, d_model, dtype, float(factor))
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = FusedEP(group, num_experts, top_k, max_tokens, d_model, dtype, factor)
        _WORKSPACES[key] = ws
    return ws


def release_workspaces():
    _WORKSPACES.clear()
