"""Mixture-of-experts feed-forward block with expert parallelism.

Semantics (no counterpart in the reference; standard top-k softmax routing):
  probs = softmax(x W_r) over E experts; the k largest are selected and weight the expert
  outputs (optionally renormalised); routed experts are gated MLPs of hidden ``expert_d_ffn``;
  ``num_shared_experts`` always-on experts are one dense gated MLP of hidden
  ``num_shared * shared_d_ffn`` applied to every token;
  out = shared(x) + sum_k w_k * expert_k(x) (+ residual);
  aux = coeff * E * sum_e f_e * P_e with f_e the fraction of token slots routed to e and P_e the
  mean router probability of e, taken over the tokens this rank routes: the micro-batch of a data-parallel
  rank, and under sequence parallelism this rank's token shard of it (the layer's loss is then the mean of
  the shards' losses, identical on every tensor-parallel rank).

Execution. Token slots are sorted by expert into a buffer whose per-expert segments are padded
to the GEMM's 128-row tile, so the grouped tcgen05 GEMM picks the expert weight per M tile
from a small device table (no host synchronisation when experts are local). With expert
parallelism the slots first cross the EP group with an all-to-all whose split sizes are the
per-rank expert counts; the inverse all-to-all brings expert outputs back, and the slot
outputs are combined with the router weights. Dropless (no capacity factor).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..layers.activations import Activation
from ..layers.mlp import MLP
from ..ops import functional as OF
from ..ops import kernels, native
from ..parallel import collectives as C
from ..parallel import mesh

TILE = 128


class _GroupedLinear(torch.autograd.Function):
    """y[rows of expert e] = x[rows of expert e] @ W[e] on the padded, expert-sorted layout."""

    @staticmethod
    def forward(ctx, xp, weight, tile_expert, k_offsets):
        e, k, n = weight.shape
        y = kernels.gemm(xp, weight, a_major=0, b_major=1, m=xp.shape[0], n=n, k=k, group_mode=1, num_groups=e,
                         group_table=tile_expert, b_group_stride=k * n)
        ctx.save_for_backward(xp, weight, tile_expert, k_offsets)
        return y

    @staticmethod
    def backward(ctx, dy):
        xp, weight, tile_expert, k_offsets = ctx.saved_tensors
        e, k, n = weight.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = kernels.gemm(dy, weight, a_major=0, b_major=0, m=dy.shape[0], n=k, k=n, group_mode=1, num_groups=e,
                              group_table=tile_expert, b_group_stride=k * n)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                kernels.gemm(xp, dy, a_major=1, b_major=1, m=k, n=n, k=xp.shape[0], group_mode=2, num_groups=e,
                             group_table=k_offsets, out=main_grad, residual=main_grad, out_dtype=main_grad.dtype)
                weight.grad_ready = True
            else:
                dw = kernels.gemm(xp, dy, a_major=1, b_major=1, m=k, n=n, k=xp.shape[0], group_mode=2, num_groups=e,
                                  group_table=k_offsets)
        return dx, dw, None, None


def grouped_linear(xp: torch.Tensor, weight: torch.Tensor, tile_expert: torch.Tensor, seg_offsets: torch.Tensor,
                   counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """xp: [P, K] expert-sorted rows with 128-padded segments; weight: [E, K, N];
    tile_expert: int32 [P/128] expert of each tile (-1 = unused tile); seg_offsets: int32 [E+1]."""
    if OF.use_native(xp):
        return _GroupedLinear.apply(xp, weight, tile_expert, seg_offsets)
    outs = torch.zeros((xp.shape[0], weight.shape[2]), dtype=xp.dtype, device=xp.device)
    off = seg_offsets.tolist()
    for e in range(weight.shape[0]):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            outs[lo:hi] = xp[lo:hi] @ weight[e]
    return outs


def padded_layout(expert_ids: torch.Tensor, num_experts: int, capacity_rows: int):
    """For slot->expert ids (any order) compute the destination row of every slot in the
    expert-sorted, 128-padded buffer. Returns (dest_row [S], seg_offsets int32 [E+1],
    tile_expert int32 [capacity_rows/128], counts [E]). All on device, no synchronisation."""
    s = expert_ids.numel()
    counts = torch.bincount(expert_ids, minlength=num_experts)
    padded = (counts + TILE - 1) // TILE * TILE
    seg_end = torch.cumsum(padded, 0)
    seg_start = seg_end - padded
    order = torch.argsort(expert_ids, stable=True)
    sorted_e = expert_ids[order]
    first_of_expert = torch.cumsum(counts, 0) - counts
    rank_in_expert = torch.arange(s, device=expert_ids.device) - first_of_expert[sorted_e]
    dest_sorted = seg_start[sorted_e] + rank_in_expert
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    seg_offsets = torch.cat([seg_start[:1] * 0, seg_end]).to(torch.int32)
    tiles = capacity_rows // TILE
    tile_start = torch.arange(tiles, device=expert_ids.device) * TILE
    tile_expert = torch.bucketize(tile_start, seg_end, right=True)
    tile_expert = torch.where(tile_expert < num_experts, tile_expert, torch.full_like(tile_expert, -1))
    # tiles inside an expert's segment but beyond its real rows still belong to it (padding rows are zero)
    return dest, seg_offsets, tile_expert.to(torch.int32), counts


native.register("icb_router_fwd", [native.P, native.I, native.I, native.I, native.I, native.P, native.P, native.P,
                                   native.P, native.P, native.P])
native.register("icb_router_bwd", [native.P, native.P, native.P, native.P, native.P, native.F, native.I, native.I,
                                   native.I, native.I, native.P, native.P])


class _Router(torch.autograd.Function):
    """Router on the native kernels: logits from the tcgen05 GEMM (fp32 output), then one kernel for softmax,
    top-k, the expert-load histogram and the mean routing probabilities; backward is one kernel plus the two
    small GEMMs of the router weight. Returns (weights [T, k] fp32, expert ids [T, k] int64, aux loss)."""

    @staticmethod
    def forward(ctx, x, weight, top_k: int, normalize: bool, aux_coeff: float):
        t, e = x.shape[0], weight.shape[0]
        logits = kernels.mm_nt(x, weight, out_dtype=torch.float32)
        probs = torch.empty((t, e), dtype=torch.float32, device=x.device)
        w = torch.empty((t, top_k), dtype=torch.float32, device=x.device)
        idx = torch.empty((t, top_k), dtype=torch.int32, device=x.device)
        counts = torch.zeros(e, dtype=torch.int32, device=x.device)
        psum = torch.zeros(e, dtype=torch.float32, device=x.device)
        native.call("icb_router_fwd", native.ptr(logits), t, e, int(top_k), 1 if normalize else 0, native.ptr(probs),
                    native.ptr(w), native.ptr(idx), native.ptr(counts), native.ptr(psum), native.stream_ptr())
        aux = (aux_coeff * e / (float(t) * top_k * t)) * (counts.float() * psum).sum()
        ctx.save_for_backward(x, weight, probs, idx, counts)
        ctx.cfg = (int(top_k), bool(normalize), float(aux_coeff))
        idx64 = idx.long()
        ctx.mark_non_differentiable(idx64)
        return w, idx64, aux

    @staticmethod
    def backward(ctx, dw, _didx, daux):
        x, weight, probs, idx, counts = ctx.saved_tensors
        top_k, normalize, aux_coeff = ctx.cfg
        t, e = probs.shape
        dw = torch.zeros((t, top_k), dtype=torch.float32, device=x.device) if dw is None else dw.contiguous().float()
        daux_t = daux.reshape(1).float().contiguous() if daux is not None else None
        dlogits = torch.empty_like(probs)
        native.call("icb_router_bwd", native.ptr(probs), native.ptr(dw), native.ptr(idx), native.ptr(counts),
                    native.ptr(daux_t), aux_coeff * e / (float(t) * t * top_k), t, e, top_k, 1 if normalize else 0,
                    native.ptr(dlogits), native.stream_ptr())
        dl = dlogits.to(x.dtype)
        dx = kernels.mm_nn(dl, weight) if ctx.needs_input_grad[0] else None       # [T, E] @ [E, d]
        dwt = kernels.mm_tn(dl, x) if ctx.needs_input_grad[1] else None           # [T, E]^T @ [T, d]
        return dx, dwt, None, None, None


class MoEBlock(nn.Module):
    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        m = config.model
        moe = m.moe
        self.d_model = m.d_model
        self.num_experts = moe.num_experts
        self.top_k = moe.top_k
        self.aux_coeff = moe.aux_loss_coeff
        self.capacity_factor = float(getattr(moe, "capacity_factor", 0.0) or 0.0)   # 0 = dropless
        self.normalize = moe.normalize_topk
        self.ffn = moe.expert_d_ffn or m.d_ffn
        self.tp_group = mesh.get_tensor_model_parallel_group()
        tp = mesh.get_tensor_model_parallel_world_size()
        self.sp_size = tp if (tp > 1 and mesh.sequence_parallel_enabled()) else 1
        self.ep_group = mesh.get_expert_model_parallel_group()
        self.ep = mesh.get_expert_model_parallel_world_size()
        self.ep_rank = mesh.get_expert_model_parallel_rank()
        if self.num_experts % self.ep:
            raise ValueError("num_experts must be divisible by the expert parallel size")
        self.e_local = self.num_experts // self.ep
        self.activation = Activation(m.activation_type)
        mult = 2 if self.activation.gated else 1
        self.router = nn.Linear(m.d_model, self.num_experts, bias=False, dtype=dtype, device=device)
        # stored [in, out] like every other linear: router.weight is [E, d] (nn.Linear) and applied as x @ W^T
        self.experts_up = nn.Parameter(torch.empty(self.e_local, m.d_model, self.ffn * mult, dtype=dtype, device=device))
        self.experts_down = nn.Parameter(torch.empty(self.e_local, self.ffn, m.d_model, dtype=dtype, device=device))
        self.experts_up.expert_parallel = True
        self.experts_down.expert_parallel = True
        self.fused_ep = None          # set lazily on the first CUDA forward (symmetric-memory workspace)
        self._fused_ep_tried = False
        self._max_tokens = config.trainer.micro_batch_size * m.max_seq_len
        self.shared = None
        if moe.num_shared_experts > 0:
            s_ffn = (moe.shared_expert_d_ffn or self.ffn) * moe.num_shared_experts
            self.shared = MLP(m.d_model, s_ffn, m.activation_type, bias=False, dropout=0.0, dtype=dtype, device=device)
        # Qwen-MoE layout: the shared expert's output is scaled per token by sigmoid(x . g)
        self.shared_gate = None
        if self.shared is not None and getattr(moe, "shared_expert_gate", False):
            self.shared_gate = nn.Linear(m.d_model, 1, bias=False, dtype=dtype, device=device)

    # ------------------------------------------------------------------ routing
    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        e = self.num_experts
        if OF.use_native(x) and x.dim() == 2 and e <= 256 and e % 8 == 0 and self.top_k <= 8 and x.shape[1] % 8 == 0 \
                and self.router.weight.dtype == x.dtype:
            return _Router.apply(x.contiguous(), self.router.weight, self.top_k, self.normalize, self.aux_coeff)
        logits = F.linear(x, self.router.weight).float()
        probs = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(probs, self.top_k, dim=-1)
        if self.normalize:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        t = x.shape[0]
        f = torch.bincount(idx.reshape(-1), minlength=self.num_experts).float() / float(t * self.top_k)
        p_mean = probs.mean(0)
        aux = self.aux_coeff * self.num_experts * (f.detach() * p_mean).sum()
        return w, idx, aux

    # ------------------------------------------------------------------ expert compute on sorted slots
    def _experts(self, xs: torch.Tensor, local_expert: torch.Tensor) -> torch.Tensor:
        """xs: [S, d] slot inputs, local_expert: [S] ids in [0, e_local). Returns [S, d]."""
        s = xs.shape[0]
        cap = (s + self.e_local * (TILE - 1) + TILE - 1) // TILE * TILE
        dest, seg_offsets, tile_expert, _counts = padded_layout(local_expert, self.e_local, cap)
        xp = torch.zeros((cap, xs.shape[1]), dtype=xs.dtype, device=xs.device)
        xp = xp.index_copy(0, dest, xs)
        h = grouped_linear(xp, self.experts_up, tile_expert, seg_offsets)
        # rows of unused tiles are never written by the grouped GEMM: the activation is told where they start
        h = self.activation(h, seg_offsets[-1:] if OF.use_native(h) else None)
        yp = grouped_linear(h, self.experts_down, tile_expert, seg_offsets)
        return yp.index_select(0, dest)

    def _experts_on_layout(self, xp, seg_offsets, tile_expert):
        """Expert MLPs on rows that already sit in the padded, expert-sorted layout."""
        h = grouped_linear(xp, self.experts_up, tile_expert, seg_offsets)
        h = self.activation(h, seg_offsets[-1:])
        return grouped_linear(h, self.experts_down, tile_expert, seg_offsets)

    def _fused_workspace(self, x):
        if not self._fused_ep_tried:
            self._fused_ep_tried = True
            if x.is_cuda and self.ep > 1 and OF.use_native(x):
                from ..parallel.fused_moe import get_fused_ep

                self.fused_ep = get_fused_ep(self.ep_group, self.num_experts, self.top_k,
                                             max(self._max_tokens, x.shape[0]), self.d_model, x.dtype,
                                             factor=float(getattr(self, "capacity_factor", 0.0) or 0.0))
        return self.fused_ep

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        """x: [T, d] -> ([T, d], aux loss)."""
        t, d = x.shape
        w, idx, aux = self.route(x)
        if self.sp_size > 1:
            # Under sequence parallelism this rank routes its token shard only: the layer's balance loss is the
            # mean of the shards' losses. The sum over the tensor-parallel group makes the value the same on
            # every rank; its backward pass is the identity, and the gradients of the replicated router weight
            # are summed over the group by the optimizer engine, so each shard's loss counts once, not tp times.
            aux = C.reduce_from_tp(aux / self.sp_size, self.tp_group)
        ws = self._fused_workspace(x) if self.ep > 1 else None
        if ws is not None and t <= ws.max_tokens:
            # dispatch, expert GEMMs and combine without leaving the device: the exchange runs inside kernels
            from ..parallel.fused_moe import fused_combine, fused_dispatch

            expert = idx.reshape(-1).to(torch.int32)
            xp, dest, seg, tile_expert, counts = fused_dispatch(x, expert, ws)
            yp = self._experts_on_layout(xp, seg, tile_expert)
            out = fused_combine(yp, w, expert, dest, counts, ws)
            if self.shared is not None:
                out = out + self._shared_out(x)
            if residual is not None:
                out = out + residual
            return out, aux
        slots_expert = idx.reshape(-1)                                   # [T*k]
        token_of_slot = torch.arange(t, device=x.device).repeat_interleave(self.top_k)
        xs = x.index_select(0, token_of_slot)
        if self.ep == 1:
            ys = self._experts(xs, slots_expert)
        else:
            # sort slots by destination rank, exchange, run local experts, exchange back
            dest_rank = slots_expert // self.e_local
            order = torch.argsort(dest_rank, stable=True)
            send_counts = torch.bincount(dest_rank, minlength=self.ep)
            recv_counts = torch.empty_like(send_counts)
            if x.is_cuda:
                dist.all_to_all_single(recv_counts, send_counts, group=self.ep_group)
            else:
                self._exchange_counts(send_counts, recv_counts)
            in_splits = send_counts.tolist()
            out_splits = recv_counts.tolist()
            xs_sorted = xs.index_select(0, order)
            e_sorted = (slots_expert.index_select(0, order) % self.e_local)
            xr = C.all_to_all(xs_sorted, out_splits, in_splits, self.ep_group)
            er = C.all_to_all_single(e_sorted.contiguous(), out_splits, in_splits, self.ep_group)
            yr = self._experts(xr, er)
            ys_sorted = C.all_to_all(yr, in_splits, out_splits, self.ep_group)
            ys = torch.empty_like(ys_sorted)
            ys = ys.index_copy(0, order, ys_sorted)
        out = (ys.view(t, self.top_k, d) * w.to(ys.dtype).unsqueeze(-1)).sum(1)
        if self.shared is not None:
            out = out + self._shared_out(x)
        if residual is not None:
            out = out + residual
        return out, aux

    def _shared_out(self, x: torch.Tensor) -> torch.Tensor:
        y = self.shared(x)
        if self.shared_gate is not None:
            y = y * torch.sigmoid(self.shared_gate(x))
        return y

    def _exchange_counts(self, send_counts, recv_counts):
        gathered = [torch.empty_like(send_counts) for _ in range(self.ep)]
        dist.all_gather(gathered, send_counts, group=self.ep_group)
        for r in range(self.ep):
            recv_counts[r] = gathered[r][self.ep_rank]


def moe_reference(x, router_w, experts_up, experts_down, top_k, activation: str, normalize: bool = False):
    """Dense per-token restatement (every token through its k experts one by one); oracle for tests."""
    from ..ops.reference import act_reference, glu_reference
    from ..ops.functional import is_gated

    probs = torch.softmax((x @ router_w.t()).float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if normalize:
        w = w / w.sum(-1, keepdim=True)
    out = torch.zeros_like(x, dtype=torch.float32)
    for e in range(experts_up.shape[0]):
        mask = (idx == e)
        if not mask.any():
            continue
        tok, slot = mask.nonzero(as_tuple=True)
        h = x[tok].float() @ experts_up[e].float()
        h = glu_reference(h, activation) if is_gated(activation) else act_reference(h, activation)
        y = h @ experts_down[e].float()
        out.index_add_(0, tok, y * w[tok, slot].unsqueeze(-1))
    return out
