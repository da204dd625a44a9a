"""Fused compute+collective paths of tensor parallelism with sequence parallelism.

``FusedTP`` owns the symmetric-memory workspaces shared by every layer of a model:

* gather scratch    : two (call-parity) gathered activation buffers ``[M, d]`` plus the per-128-row
  arrival counters that the peers bump when their pushed shard chunks have landed, used by
  ``icb_ag_gemm`` (all-gather -> GEMM in one kernel) for gathers that live for one call (the output
  gradients of row-parallel layers);
* gather slots      : one persistent gathered buffer ``[M, d]`` with its own counters per column-parallel
  call site. The forward gather of a call site stays in its slot until the weight gradient of the same
  call site has used it, so nothing is cloned; and a slot can be filled by the *producer* of its rows;
* scatter workspace : two receive buffers ``[t][M/t][d]`` plus per-tile arrival counters used by
  ``icb_gemm_rs`` (GEMM -> reduce-scatter in one kernel).

Forward and backward of the column- / row-parallel linears map onto these kernels:

  column fwd  : AG(x) -> GEMM                      (icb_ag_gemm, a_major 0)
  column wgrad: gathered(x)^T GEMM dy              (plain GEMM on the slot the forward filled; runs before
                                                    the dgrad so that no peer can refill the slot early)
  column dgrad: GEMM(dy, W^T) -> RS                (icb_gemm_rs)
  row fwd     : GEMM -> RS (+bias +residual)       (icb_gemm_rs)
  row fwd + next norm : GEMM -> RS -> RMSNorm -> push into the next column call site's slot
                                                   (icb_gemm_rs_norm_ag; the consumer runs icb_ag_gemm with
                                                    the "pushed by the producers" flag and only waits)
  column dgrad + norm bwd : GEMM(dy, W^T) -> RS -> RMSNorm backward (+ residual gradient) -> push into the scratch
                                                   gather buffer of the row-parallel dgrad that follows
                                                   (icb_gemm_rs_norm_bwd_ag; mirror of the forward boundary)
  row dgrad   : AG(dy) -> GEMM                     (icb_ag_gemm, a_major 0, scratch buffer)
  row wgrad   : x^T GEMM gathered(dy)              (plain GEMM on the scratch buffer the dgrad call filled)

Every rank must issue the same sequence of calls (SPMD). Each buffer counts its calls in a device word
that the kernels read as the epoch of their cumulative flags, so a captured CUDA graph replays
correctly; the host-side counter only selects the parity of the scratch / receive buffers, which is
why a captured region must contain an even number of calls per parity workspace (checked by the
trainer). The ``torch.distributed`` path in :mod:`ironcore_b200.parallel.tensor_parallel` is the
fallback and the oracle.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import kernels, native
from ..ops.native import call, dtype_code, ptr, stream_ptr
from .symmetric import SymmetricBuffer, nvls_requested, symmetric_memory_available

P, I, L, F = native.P, native.I, native.L, native.F
native.register("icb_ag_gemm", [P, P, P, P, P, I, I, I, I, P, P, P, P, P, I, L, L, L, I, I, I, I, P, P, P, I])
native.register("icb_gemm_rs", [P, P, P, P, P, I, I, I, L, L, L, L, I, I, P, P, P, P, I, I, P, P, P, P])
native.register("icb_gemm_rs_norm_ag", [P, P, P, P, P, I, I, I, L, L, L, L, I, I, P, P, P, P, I, I, P, P, P, P,
                                        P, F, F, P, P, P, P])
native.register("icb_gemm_rs_norm_bwd_ag", [P, P, P, P, I, I, I, L, L, L, L, I, I, P, P, P, P, I, I, P, P, P, P,
                                            P, F, P, P, L, P, P, P, P])


class GatherSlot:
    """One gathered activation buffer ``[tokens, width]`` of a symmetric allocation with the arrival
    counters of its 128-row blocks and the device word that counts its completed gathers."""

    def __init__(self, sbuf: SymmetricBuffer, data_off: int, ready_off: int, tokens: int, width: int, dtype, rank: int,
                 rows: int, index: int):
        self.index = index
        self.data_off = data_off
        self.buf = sbuf.view(data_off, (tokens, width), dtype)
        self.local = self.buf[rank * rows:(rank + 1) * rows]
        self.peers = sbuf.peer_table(data_off)
        self.peer_ready = sbuf.peer_table(ready_off)
        self.ready = sbuf.view(ready_off, (tokens // 128,), torch.int32)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=sbuf.local.device)
        self.mc = (sbuf.multicast_ptr + data_off) if sbuf.multicast_ptr else 0


def row_width_supported(width: int) -> bool:
    """The fused reduce-scatter + norm producer publishes whole 8 KiB chunks: a row must divide a chunk
    or be a multiple of it."""
    row_bytes = width * 2
    return row_bytes % 8192 == 0 if row_bytes >= 8192 else 8192 % row_bytes == 0


class FusedTP:
    def __init__(self, tokens: int, width: int, group, dtype=torch.bfloat16, nvls: Optional[bool] = None,
                 num_slots: int = 0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.tokens, self.width, self.dtype = tokens, width, dtype
        if tokens % self.world or (tokens // self.world) % 128 or width % 32:
            raise ValueError("fused TP needs tokens/world to be a multiple of 128 and width a multiple of 32")
        self.rows = tokens // self.world
        es = 2
        self.max_n_tiles = (width + 255) // 256
        # ---- gather workspace: two scratch buffers by call parity, then the persistent slots ----
        g_data = tokens * width * es
        ready_bytes = ((tokens // 128) * 4 + 255) // 256 * 256
        n_bufs = 2 + num_slots
        self._g_off = [i * g_data for i in range(n_bufs)]
        ready_off = [n_bufs * g_data + i * ready_bytes for i in range(1 + num_slots)]   # scratch shares one array
        g_total = ready_off[-1] + ready_bytes
        self.gbuf = SymmetricBuffer(g_total, group)
        dev = self.gbuf.local.device
        self.g_views = [self.gbuf.view(self._g_off[p], (tokens, width), dtype) for p in range(2)]
        self.g_peers = [self.gbuf.peer_table(self._g_off[p]) for p in range(2)]
        self.g_peer_ready = self.gbuf.peer_table(ready_off[0])
        self.g_ready = self.gbuf.view(ready_off[0], (tokens // 128,), torch.int32)
        self.g_epoch = 0
        self.g_epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.slots: List[GatherSlot] = [
            GatherSlot(self.gbuf, self._g_off[2 + i], ready_off[1 + i], tokens, width, dtype, self.rank, self.rows, i)
            for i in range(num_slots)]
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
        self.r_epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        # True: forward keeps the gathered activations (32 MiB at 4096 x 4096) for the weight gradient;
        # False: backward re-gathers inside the wgrad kernel (less memory, exposed transfer).
        self.save_gathered = True
        # NVLS: push the gathered shard once with multimem.st and reduce the scattered partials with
        # multimem.ld_reduce when the symmetric allocations have a multicast mapping on every rank.
        have = torch.tensor([1 if (self.gbuf.multicast_ptr and self.rbuf.multicast_ptr) else 0],
                            dtype=torch.int32, device=dev)
        if self.world > 1:
            dist.all_reduce(have, op=dist.ReduceOp.MIN, group=group)
        have = self.world > 1 and int(have.item()) == 1
        self.nvls_ag = bool(have and (nvls_requested(self.world, "ag") if nvls is None else nvls))
        # Whether the four epilogue warps of every CTA push chunks of the gather shard before their first
        # accumulator is ready, next to the two copy warps. Measured level (4 ranks: 0.190 ms against 0.195 ms for
        # the qkv projection; the shard takes about 50 us to land either way, which is the fabric's time for
        # 24 MB into every GPU, not the warps') and 3 % slower at 2 ranks: off.
        self.push_helpers = False
        self.nvls_rs = bool(have and (nvls_requested(self.world, "rs") if nvls is None else nvls))
        self.nvls = self.nvls_ag or self.nvls_rs
        self.norm_fusable = row_width_supported(width)

    # ------------------------------------------------------------------ raw kernels
    def ag_gemm(self, x_shard: torch.Tensor, b: torch.Tensor, *, a_major: int, b_major: int, n: int,
                bias=None, out=None, residual=None, out_dtype=None, slot: Optional[GatherSlot] = None,
                pushed: bool = False) -> torch.Tensor:
        """AG(x_shard) (x) b. a_major 0: [tokens, width] @ b -> [tokens, n];
        a_major 1: gathered^T @ b[tokens, n] -> [width, n].
        ``slot``: gather into this persistent buffer instead of the parity scratch. ``pushed``: every rank's
        rows were (or are being) written into the slot by their producers (``gemm_rs(..., norm=...)``); the
        kernel pushes nothing and waits for the slot's counters."""
        if x_shard.shape != (self.rows, self.width) or x_shard.dtype != self.dtype:
            raise ValueError(f"fused gather expects a [{self.rows}, {self.width}] {self.dtype} shard")
        if slot is None:
            self.g_epoch += 1
            par = self.g_epoch & 1
            gathered, peers, peer_ready, ready, epoch_dev = (self.g_views[par], self.g_peers[par], self.g_peer_ready,
                                                             self.g_ready, self.g_epoch_dev)
            mc = (self.gbuf.multicast_ptr + self._g_off[par]) if self.nvls_ag else None
        else:
            gathered, peers, peer_ready, ready, epoch_dev = slot.buf, slot.peers, slot.peer_ready, slot.ready, \
                slot.epoch_dev
            mc = slot.mc if (self.nvls_ag and slot.mc) else None
        if not pushed:
            local = gathered[self.rank * self.rows:(self.rank + 1) * self.rows]
            if local.data_ptr() != x_shard.data_ptr():
                local.copy_(x_shard)
        m = self.tokens if a_major == 0 else self.width
        out_dtype = out_dtype or (out.dtype if out is not None else self.dtype)
        if out is None:
            out = torch.empty((m, n), dtype=out_dtype, device=x_shard.device)
        ldr = residual.stride(0) if residual is not None else 0
        call("icb_ag_gemm", ptr(gathered), ptr(peers), ptr(peer_ready), None, ptr(ready), self.rank, self.world,
             self.rows, self.width, ptr(epoch_dev), ptr(b), ptr(out), ptr(bias), ptr(residual), int(n), b.stride(0),
             out.stride(0), ldr, int(a_major), int(b_major), dtype_code(self.dtype),
             1 if out_dtype == torch.float32 else 0, ptr(native.status_tensor(x_shard.device)), stream_ptr(), mc,
             1 if pushed else (2 if self.push_helpers else 0))
        epoch_dev.add_(1)
        self.last_gathered = gathered
        return out

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, *, b_major: int, bias=None, residual=None, norm=None):
        """reduce_scatter_rows(a[tokens, k] (x) b) -> [tokens / world, width].
        ``norm = (gamma, eps, w_offset, slot)``: the same kernel also RMS-normalises the reduced rows and stores
        them into every rank's copy of ``slot``; returns ``(out, rstd)`` and ``slot.local`` holds this rank's
        normalised rows."""
        if a.shape[0] != self.tokens or a.dtype != self.dtype:
            raise ValueError("fused reduce-scatter expects the full token dimension")
        n = self.width
        k = a.shape[1]
        self.r_epoch += 1
        par = self.r_epoch & 1
        out = torch.empty((self.rows, n), dtype=self.dtype, device=a.device)
        ldr = residual.stride(0) if residual is not None else 0
        recv_ptr = self.rbuf.local.data_ptr() + self._r_off[par]
        common = (ptr(a), ptr(b), ptr(out), ptr(bias), ptr(residual), self.tokens, n, k, a.stride(0),
                  b.stride(0), out.stride(0), ldr, int(b_major), dtype_code(self.dtype), ptr(self.r_peers[par]),
                  ptr(self.r_peer_flags), recv_ptr, ptr(self.r_flags), self.rank, self.world, ptr(self.r_epoch_dev),
                  ptr(native.status_tensor(a.device)), stream_ptr(),
                  (self.rbuf.multicast_ptr + self._r_off[par]) if self.nvls_rs else None)
        if norm is None:
            call("icb_gemm_rs", *common)
            self.r_epoch_dev.add_(1)
            return out
        gamma, eps, w_offset, slot = norm
        if not self.norm_fusable:
            raise ValueError(f"width {self.width} is not supported by the fused reduce-scatter + norm kernel")
        rstd = torch.empty(self.rows, dtype=torch.float32, device=a.device)
        call("icb_gemm_rs_norm_ag", *common, ptr(gamma), float(eps), float(w_offset), ptr(rstd), ptr(slot.peers),
             slot.mc if (self.nvls_ag and slot.mc) else None, ptr(slot.peer_ready))
        self.r_epoch_dev.add_(1)
        return out, rstd

    def gemm_rs_norm_bwd(self, a: torch.Tensor, b: torch.Tensor, *, b_major: int, residual, gamma, w_offset: float,
                         rstd: torch.Tensor, x: torch.Tensor):
        """Backward of a ``gemm_rs(..., norm=...)`` boundary: ``dn = reduce_scatter_rows(a @ b)`` is the gradient
        of the normalised rows; returns ``(dx, dn)`` with ``dx = rmsnorm_backward(dn; x, rstd, gamma) + residual``
        and leaves every rank's ``dx`` rows in the scratch gather buffer that the NEXT scratch ``ag_gemm`` call
        uses (call it with ``pushed=True``)."""
        if a.shape[0] != self.tokens or a.dtype != self.dtype or not self.norm_fusable:
            raise ValueError("fused reduce-scatter + norm backward: unsupported operand")
        n, k = self.width, a.shape[1]
        self.r_epoch += 1
        par = self.r_epoch & 1
        gpar = (self.g_epoch + 1) & 1          # parity of the scratch gather buffer the next ag_gemm call takes
        out = torch.empty((self.rows, n), dtype=self.dtype, device=a.device)
        dn = torch.empty((self.rows, n), dtype=self.dtype, device=a.device)
        ldr = residual.stride(0) if residual is not None else 0
        recv_ptr = self.rbuf.local.data_ptr() + self._r_off[par]
        mc = (self.gbuf.multicast_ptr + self._g_off[gpar]) if self.nvls_ag else None
        call("icb_gemm_rs_norm_bwd_ag", ptr(a), ptr(b), ptr(out), ptr(residual), self.tokens, n, k, a.stride(0),
             b.stride(0), out.stride(0), ldr, int(b_major), dtype_code(self.dtype), ptr(self.r_peers[par]),
             ptr(self.r_peer_flags), recv_ptr, ptr(self.r_flags), self.rank, self.world, ptr(self.r_epoch_dev),
             ptr(native.status_tensor(a.device)), stream_ptr(),
             (self.rbuf.multicast_ptr + self._r_off[par]) if self.nvls_rs else None, ptr(gamma), float(w_offset),
             ptr(rstd), ptr(x), x.stride(0), ptr(dn), ptr(self.g_peers[gpar]), mc, ptr(self.g_peer_ready))
        self.r_epoch_dev.add_(1)
        return out, dn

    # ------------------------------------------------------------------ autograd entry points
    def row_norm_column(self, x, w_row, b_row, residual, gamma, eps: float, w_offset: float, w_col, b_col,
                        slot: GatherSlot):
        """``h = reduce_scatter(x @ w_row) + b_row + residual`` ; ``y = all_gather(rmsnorm(h)) @ w_col + b_col``
        as two kernels in forward (producer pushes, consumer only waits) and the mirrored pair in backward.
        Returns ``(h, y)``."""
        return _RowNormColumn.apply(x, w_row, b_row, residual, gamma, w_col, b_col, self, slot, float(eps),
                                    float(w_offset))

    def allgather_linear(self, x_shard, weight, bias=None, slot: Optional[GatherSlot] = None, pushed: bool = False):
        return _AllGatherLinear.apply(x_shard, weight, bias, self, slot, pushed)

    def linear_reduce_scatter(self, x, weight, bias=None, residual=None):
        return _LinearReduceScatter.apply(x, weight, bias, residual, self)

    def linear_reduce_scatter_norm(self, x, weight, bias, residual, gamma, eps: float, w_offset: float,
                                   slot: GatherSlot):
        """Row-parallel linear + residual, then RMSNorm of the result pushed into ``slot`` on every rank.
        Returns ``(h, normed)``: the residual-stream shard and this rank's normalised rows (a view of the slot,
        to be handed to the column-parallel linear that owns the slot with ``pushed=True``)."""
        return _LinearRSNorm.apply(x, weight, bias, residual, gamma, self, slot, float(eps), float(w_offset))

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
    def forward(ctx, x_shard, weight, bias, ws: FusedTP, slot, pushed):
        x2 = x_shard.reshape(-1, x_shard.shape[-1])
        if not pushed:
            x2 = x2.contiguous()
        y = ws.ag_gemm(x2, weight, a_major=0, b_major=1, n=weight.shape[1], bias=bias, slot=slot, pushed=pushed)
        # The weight gradient needs the gathered activations. A slot keeps them until this call site runs
        # again; what protects it from an early refill by a fast peer is the reduce-scatter of the input
        # gradient, issued after the weight gradient below: a peer cannot finish its backward pass, and
        # start the next forward, before it has received this rank's partial tiles. Without an input
        # gradient there is no such reduce-scatter, and the scratch buffer is reused two calls later:
        # both cases keep a private copy. (A re-gather inside the wgrad kernel cannot hide its transfer:
        # the reduction runs over the gathered rows, so every output tile needs all of them at once.)
        # The slot is kept as a plain attribute, not through save_for_backward: every buffer of the
        # workspace is a view of one symmetric allocation and shares its version counter, so autograd
        # would take any later gather into a neighbouring buffer for a modification of this one.
        ctx.slot_gathered = None
        if not ws.save_gathered:
            x_full = x2
        elif slot is not None and ctx.needs_input_grad[0]:
            ctx.slot_gathered = slot.buf
            x_full = None
        else:
            x_full = ws.last_gathered.clone()
        ctx.save_for_backward(x_full, weight)
        ctx.ws = ws
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        if ctx.slot_gathered is not None:
            x2 = ctx.slot_gathered
        ws: FusedTP = ctx.ws
        dy = dy.contiguous()
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
        dx = ws.gemm_rs(dy, weight, b_major=0) if ctx.needs_input_grad[0] else None
        db = dy.sum(0, dtype=torch.float32).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None, None, None


def _row_parallel_backward(ctx, x2, weight, dy_shard, ws: FusedTP):
    """dX_local = AG(dy) @ W^T ; the gathered dy stays in the scratch buffer for the weight gradient."""
    dx = ws.ag_gemm(dy_shard, weight, a_major=0, b_major=0, n=weight.shape[0])
    dy_full = ws.last_gathered
    dw = None
    if ctx.needs_input_grad[1]:
        def compute(acc):
            if acc is not None:
                return kernels.mm_tn(x2, dy_full, out=acc, residual=acc, out_dtype=acc.dtype)
            return kernels.mm_tn(x2, dy_full)

        dw = _accumulate_or_return(weight, compute)
    db = dy_shard.sum(0, dtype=torch.float32).to(dy_shard.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
    return dx, dw, db


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
        dy_shard = dy_shard.contiguous()
        dx, dw, db = _row_parallel_backward(ctx, x2, weight, dy_shard, ctx.ws)
        dres = dy_shard if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, None


class _LinearRSNorm(torch.autograd.Function):
    """h = reduce_scatter(x @ W) + bias + residual ; normed = rmsnorm(h) * (gamma + w_offset), written into the
    gather slot of the following column-parallel linear on every rank by the same kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, gamma, ws: FusedTP, slot, eps, w_offset):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        res2 = residual.reshape(-1, weight.shape[1]).contiguous() if residual is not None else None
        h, rstd = ws.gemm_rs(x2, weight, b_major=1, bias=bias, residual=res2, norm=(gamma, eps, w_offset, slot))
        ctx.save_for_backward(x2, weight, h, rstd, gamma)
        ctx.ws = ws
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.w_offset = w_offset
        return h, slot.buf.narrow(0, ws.rank * ws.rows, ws.rows)

    @staticmethod
    def backward(ctx, dh, dnormed):
        x2, weight, h, rstd, gamma = ctx.saved_tensors
        dgamma = None
        if dnormed is not None:
            dres_in = dh.contiguous() if dh is not None else None
            dh, dg, _ = kernels.norm_bwd(dnormed.contiguous(), h, gamma, None, rstd, True, False, dres_in=dres_in,
                                         w_offset=ctx.w_offset)
            dgamma = dg.to(gamma.dtype)
        dh = dh.contiguous()
        dx, dw, db = _row_parallel_backward(ctx, x2, weight, dh, ctx.ws)
        dres = dh if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, dgamma, None, None, None, None


class _RowNormColumn(torch.autograd.Function):
    """A whole norm boundary of the sequence-parallel layer: row-parallel linear (+ residual) -> RMSNorm ->
    column-parallel linear. Forward: ``icb_gemm_rs_norm_ag`` then ``icb_ag_gemm`` (pushed). Backward: the column
    layer's weight gradient from the slot, ``icb_gemm_rs_norm_bwd_ag`` (column dgrad -> reduce-scatter -> norm
    backward + residual gradient -> gather), the gain's gradient, then the row layer's ``icb_ag_gemm`` (pushed)
    and weight gradient. The residual stream ``h`` passes through the node, so its gradient from later layers
    is an input of the fused backward kernel."""

    @staticmethod
    def forward(ctx, x, w_row, b_row, residual, gamma, w_col, b_col, ws: FusedTP, slot, eps, w_offset):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        res2 = residual.reshape(-1, w_row.shape[1]).contiguous() if residual is not None else None
        h, rstd = ws.gemm_rs(x2, w_row, b_major=1, bias=b_row, residual=res2, norm=(gamma, eps, w_offset, slot))
        y = ws.ag_gemm(slot.local, w_col, a_major=0, b_major=1, n=w_col.shape[1], bias=b_col, slot=slot, pushed=True)
        ctx.save_for_backward(x2, w_row, h, rstd, gamma, w_col)
        ctx.ws, ctx.slot_gathered, ctx.w_offset = ws, slot.buf, w_offset
        ctx.has_bias = b_row is not None          # name used by _row_parallel_backward
        ctx.has_col_bias = b_col is not None
        ctx.has_res = residual is not None
        return h, y

    @staticmethod
    def backward(ctx, dh_later, dy):
        x2, w_row, h, rstd, gamma, w_col = ctx.saved_tensors
        ws: FusedTP = ctx.ws
        dy = dy.contiguous()
        # column-parallel weight gradient first: it reads the slot, which a peer may refill once it has
        # received this rank's partial tiles of the reduce-scatter below
        dw_col = None
        if ctx.needs_input_grad[5]:
            gathered = ctx.slot_gathered

            def compute_col(acc):
                if acc is not None:
                    return kernels.mm_tn(gathered, dy, out=acc, residual=acc, out_dtype=acc.dtype)
                return kernels.mm_tn(gathered, dy)

            dw_col = _accumulate_or_return(w_col, compute_col)
        db_col = dy.sum(0, dtype=torch.float32).to(dy.dtype) if ctx.has_col_bias and ctx.needs_input_grad[6] else None
        dres_in = dh_later.contiguous() if dh_later is not None else None
        dh, dn = ws.gemm_rs_norm_bwd(dy, w_col, b_major=0, residual=dres_in, gamma=gamma, w_offset=ctx.w_offset,
                                     rstd=rstd, x=h)
        dgamma = None
        if ctx.needs_input_grad[4]:
            _, dg, _ = kernels.norm_bwd(dn, h, gamma, None, rstd, True, False, w_offset=ctx.w_offset)
            dgamma = dg.to(gamma.dtype)
        # row-parallel backward on the rows the kernel above has already gathered on every rank
        dx = ws.ag_gemm(dh, w_row, a_major=0, b_major=0, n=w_row.shape[0], pushed=True)
        dh_full = ws.last_gathered
        dw_row = None
        if ctx.needs_input_grad[1]:
            def compute_row(acc):
                if acc is not None:
                    return kernels.mm_tn(x2, dh_full, out=acc, residual=acc, out_dtype=acc.dtype)
                return kernels.mm_tn(x2, dh_full)

            dw_row = _accumulate_or_return(w_row, compute_row)
        db_row = dh.sum(0, dtype=torch.float32).to(dh.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        dres = dh if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw_row, db_row, dres, dgamma, dw_col, db_col, None, None, None, None


def attach_fused_tp(model, config) -> Optional[FusedTP]:
    """Create the shared workspaces and hand them to every sequence-parallel column / row parallel
    linear of ``model``; every fused column-parallel linear gets its own gather slot, and where a
    row-parallel linear is followed by RMSNorm and a fused column-parallel linear the pair is linked so
    that one kernel reduces, normalises and gathers (``parallel.fused_norm_gather``). Returns None (and
    leaves the NCCL path active) when symmetric memory is unavailable or the shapes do not fit the
    kernels' tiling."""
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
    head = getattr(model, "output_layer", None)
    columns, rows = [], []
    for mod in model.modules():
        if mod is head:
            continue   # keeps the number of fused calls per micro-batch even (needed for CUDA-graph replay)
        if isinstance(mod, ColumnParallelLinear) and mod.sequence_parallel and mod.in_features == width:
            columns.append(mod)
        elif isinstance(mod, RowParallelLinear) and mod.sequence_parallel and mod.out_features == width:
            rows.append(mod)
    ws = FusedTP(tokens, width, group, dtype, num_slots=len(columns))
    for i, mod in enumerate(columns):
        mod.fused = ws
        mod.gather_slot = ws.slots[i]
    for mod in rows:
        mod.fused = ws
    link = getattr(model, "link_fused_norm_gather", None)
    want = str(getattr(config.parallel, "fused_norm_gather", "auto")).lower()
    # "auto" keeps the separate kernels: on the Llama-7B layer shapes the linked form measured 11 % slower at
    # 2 ranks (half of the consumer's tiles are local and hide its own push) and level at 4 ranks (0.358 ms
    # against 0.354 ms per boundary; 61.1 k against 62.2 k tokens/s for the whole step), so it stays opt-in.
    on = want in ("on", "true", "1")
    if link is not None and on and ws.norm_fusable:
        link()
    return ws
