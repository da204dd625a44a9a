"""Muon for 2-D hidden weight matrices, in distributed form.

Per matrix:  m <- mu * m + g ;  u = g + mu * m (Nesterov) or m ;
X = NewtonSchulz5(u)  (quintic iteration in bf16 on the normalised matrix, computed on the
wide orientation):  A = X X^T ; B = b A + c A A ; X <- a X + B X   with
(a, b, c) = (3.4445, -4.7750, 2.0315);  W <- W (1 - lr wd) - lr * sqrt(max(1, fan_out/fan_in)) * X.

Fused tensors (q|k|v, gate|up) and stacked expert weights are orthogonalised per logical
matrix. Distribution: every logical matrix has an owner rank in the data-parallel group
(greedy balance by Newton-Schulz FLOPs); the owner keeps the momentum, runs the iteration
on the (TP-gathered) matrix and publishes the update once: every owner packs the updates of
its matrices into one send buffer, one all-gather over the data-parallel group delivers the
packs, and every rank adds each matrix's update from its owner's pack (wire bytes: one copy
of the Muon parameters per rank and step, against two for an all-reduce of a dense update
buffer). Momentum memory and Newton-Schulz time divide by the number of ranks. On CUDA the
three matrix products per iteration are the tcgen05 GEMM.
(No counterpart in the reference; semantics follow the published Muon optimizer.)
"""

from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.distributed as dist

from ..ops import kernels
from ..parallel import mesh as _mesh

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz_reference(g: torch.Tensor, steps: int = 5, eps: float = 1e-7, dtype=torch.bfloat16) -> torch.Tensor:
    """Plain PyTorch quintic Newton-Schulz orthogonalisation of a 2-D matrix."""
    a, b, c = NS_COEFFS
    x = g.to(dtype)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.float().norm() + eps).to(dtype)
    for _ in range(steps):
        A = x @ x.t()
        B = b * A + c * (A @ A)
        x = a * x + B @ x
    return x.t() if transposed else x


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Newton-Schulz on the native GEMM (CUDA, dims multiples of 8) or the reference path."""
    if not (g.is_cuda and g.shape[0] % 8 == 0 and g.shape[1] % 8 == 0):
        if g.is_cuda:
            from ..ops.functional import note_fallback

            note_fallback("Newton-Schulz", f"matrix {tuple(g.shape)} has a side that is not a multiple of 8")
        return newton_schulz_reference(g, steps, eps, torch.bfloat16 if g.is_cuda else torch.float32).to(g.dtype)
    a, b, c = NS_COEFFS
    x = g.to(torch.bfloat16)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t().contiguous()
    x = (x / (x.float().norm() + eps).to(torch.bfloat16)).contiguous()
    for _ in range(steps):
        A = kernels.mm_nt(x, x)                 # X X^T   (both operands K-major)
        A2 = kernels.mm_nn(A, A)                # A A
        B = (b * A + c * A2).contiguous()
        x = kernels.mm_nn(B, x, residual=(a * x).contiguous())   # B X + a X in the GEMM epilogue
    return (x.t() if transposed else x).to(g.dtype)


class _Matrix:
    __slots__ = ("slot", "group_idx", "expert", "col_lo", "col_hi", "full_shape", "owner", "momentum", "tp_dim",
                 "part", "key", "pack_off", "pack_numel")


class MuonState:
    def __init__(self, engine, config):
        self.engine = engine
        self.config = config
        o = config.optim
        self.momentum = o.muon_momentum
        self.nesterov = o.nesterov
        self.steps = o.muon_ns_steps
        self.weight_decay = o.muon_weight_decay
        self.tp_group = engine.tp_group
        self.tp_size = engine.tp_size
        self.matrices: List[_Matrix] = []
        for gi, g in enumerate(engine.groups):
            for s in g.slots:
                if g.regions[s.region].kind != "muon":
                    continue
                p = s.param
                parts = getattr(p, "tp_parts", 1)
                tp_dim = getattr(p, "tp_shard_dim", None)
                experts = range(p.shape[0]) if p.dim() == 3 else [None]
                cols = p.shape[-1]
                if isinstance(parts, int):
                    sizes = [cols // parts] * parts
                else:
                    sizes = [x // self.tp_size if tp_dim is not None and self.tp_size > 1 else x for x in parts]
                # checkpoint key: independent of the TP and EP layout (part index of a fused tensor, global
                # expert index), because the momentum is kept for the whole logical matrix
                e_base = 0
                if p.dim() == 3 and getattr(p, "expert_parallel", False):
                    e_base = _mesh.get_expert_model_parallel_rank() * p.shape[0]
                for e in experts:
                    lo = 0
                    for part, sz in enumerate(sizes):
                        mtx = _Matrix()
                        mtx.slot, mtx.group_idx, mtx.expert = s, gi, e
                        mtx.part = part
                        mtx.key = f"{s.name}|{None if e is None else e + e_base}|{part}"
                        mtx.col_lo, mtx.col_hi = lo, lo + sz
                        rows = p.shape[-2]
                        fr, fc = rows, sz
                        if tp_dim is not None and self.tp_size > 1 and p.dim() == 2:
                            if tp_dim == 0:
                                fr = rows * self.tp_size
                            else:
                                fc = sz * self.tp_size
                        mtx.full_shape = (fr, fc)
                        mtx.tp_dim = tp_dim if (self.tp_size > 1 and p.dim() == 2) else None
                        mtx.owner, mtx.momentum = 0, None
                        self.matrices.append(mtx)
                        lo += sz
        # greedy balance of Newton-Schulz cost over the reduction group of each flat group
        for gi, g in enumerate(engine.groups):
            mats = [m for m in self.matrices if m.group_idx == gi]
            load = [0.0] * max(g.dp, 1)
            for m in sorted(mats, key=lambda t: -self._cost(t.full_shape)):
                r = min(range(len(load)), key=lambda i: load[i])
                m.owner = r
                load[r] += self._cost(m.full_shape)
        # position of every matrix's (local, TP-sliced) update inside its owner's pack
        self.pack_size: List[int] = []
        for gi, g in enumerate(engine.groups):
            used = [0] * max(g.dp, 1)
            for m in self.matrices:
                if m.group_idx != gi:
                    continue
                rows = m.slot.param.shape[-2]
                m.pack_numel = rows * (m.col_hi - m.col_lo)
                m.pack_off = used[m.owner]
                used[m.owner] += (m.pack_numel + 127) // 128 * 128
            self.pack_size.append(max(used) if used else 0)

    @staticmethod
    def _cost(shape) -> float:
        r, c = min(shape), max(shape)
        return 4.0 * r * r * c + 2.0 * r * r * r

    def _view(self, buf: torch.Tensor, m: _Matrix) -> torch.Tensor:
        s = m.slot
        t = buf[s.offset:s.offset + s.numel].view(s.param.shape)
        if m.expert is not None:
            t = t[m.expert]
        return t[:, m.col_lo:m.col_hi]

    def _gather_tp(self, local: torch.Tensor, m: _Matrix) -> torch.Tensor:
        if m.tp_dim is None:
            return local
        parts = [torch.empty_like(local) for _ in range(self.tp_size)]
        dist.all_gather(parts, local.contiguous(), group=self.tp_group)
        return torch.cat(parts, dim=m.tp_dim)

    def _slice_tp(self, full: torch.Tensor, m: _Matrix) -> torch.Tensor:
        if m.tp_dim is None:
            return full
        r = dist.get_rank(self.tp_group)
        return full.chunk(self.tp_size, dim=m.tp_dim)[r]

    @torch.no_grad()
    def step(self, coef: torch.Tensor, lr: float):
        eng = self.engine
        send = []
        for gi, g in enumerate(eng.groups):
            # (zeros: the tail of a pack that is shorter than the longest one is sent but never read)
            send.append(torch.zeros(self.pack_size[gi], dtype=g.dtype, device=g.device)
                        if g.dp > 1 and self.pack_size[gi] > 0 else None)
        for m in self.matrices:
            g = eng.groups[m.group_idx]
            mine = (m.owner == g.dp_rank)
            if not mine and m.tp_dim is None:
                continue
            grad_local = self._view(g.grad_buf, m)
            if m.tp_dim is not None:
                grad_full = self._gather_tp(grad_local.contiguous(), m)  # collective: every TP rank joins
                if not mine:
                    continue
            else:
                grad_full = grad_local
            gf = grad_full.float() * (coef.to(grad_full.device) / eng.grad_div)
            if m.momentum is None:
                m.momentum = torch.zeros_like(gf)
            m.momentum.mul_(self.momentum).add_(gf)
            u = gf.add(m.momentum, alpha=self.momentum) if self.nesterov else m.momentum
            x = newton_schulz(u, self.steps)
            fan_in, fan_out = m.full_shape
            scale = math.sqrt(max(1.0, fan_out / fan_in))
            delta = self._slice_tp((-lr * scale) * x.float(), m)
            target = send[m.group_idx]
            if target is None:
                w = self._view(g.param_buf, m)
                if self.weight_decay:
                    w.mul_(1 - lr * self.weight_decay)
                w.add_(delta.to(w.dtype))
            else:
                target[m.pack_off:m.pack_off + m.pack_numel].view(delta.shape).copy_(delta.to(target.dtype))
        for gi, (g, pack) in enumerate(zip(eng.groups, send)):
            if pack is None:
                continue
            if g.device.type == "cpu":
                parts = [torch.empty_like(pack) for _ in range(g.dp)]
                dist.all_gather(parts, pack, group=g.reduce_group)
                recv = torch.stack(parts)
            else:
                recv = torch.empty(g.dp, pack.numel(), dtype=pack.dtype, device=pack.device)
                dist.all_gather_into_tensor(recv.view(-1), pack, group=g.reduce_group)
            if self.weight_decay:
                for r in g.regions:
                    if r.kind == "muon" and r.end > r.start:
                        g.param_buf[r.start:r.end].mul_(1 - lr * self.weight_decay)
            for m in self.matrices:
                if m.group_idx != gi:
                    continue
                w = self._view(g.param_buf, m)
                w.add_(recv[m.owner, m.pack_off:m.pack_off + m.pack_numel].view(w.shape))

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """Momentum of every logical matrix by layout-independent key. Collective: each momentum lives on
        its owner in the reduction group and is broadcast from there; data-parallel rank 0 (the checkpoint
        writer) keeps a host copy, the other ranks keep nothing. With expert parallelism and a merged
        (non-distributed) checkpoint the expert ranks' dictionaries are then collected on expert rank 0."""
        out: Dict[str, torch.Tensor] = {}
        eng = self.engine
        for m in self.matrices:
            g = eng.groups[m.group_idx]
            mine = m.owner == g.dp_rank
            t = m.momentum if mine else None
            if g.dp > 1:
                buf = torch.zeros(m.full_shape, dtype=torch.float32, device=g.device)
                if t is not None:
                    buf.copy_(t)
                dist.broadcast(buf, src=_mesh.global_rank_of(g.reduce_group, m.owner), group=g.reduce_group)
                t = buf
            if t is not None and g.dp_rank == 0:
                out[m.key] = t.detach().float().cpu()
        ep = _mesh.get_expert_model_parallel_world_size()
        if ep > 1 and not getattr(self.config.operation, "save_dist_ckpt", False):
            group = _mesh.get_expert_model_parallel_group()
            dst = _mesh.global_rank_of(group, 0)
            expert_keys = {m.key for m in self.matrices if m.expert is not None}
            mine_exp = {k: v for k, v in out.items() if k in expert_keys}
            parts = [None] * ep if dist.get_rank() == dst else None
            dist.gather_object(mine_exp, parts, dst=dst, group=group)
            if parts is not None:
                for d in parts:
                    out.update(d)
        return out

    def load_state_dict(self, sd: Dict[str, torch.Tensor]):
        """Owners take the momenta of their matrices; everything else in ``sd`` is ignored."""
        for m in self.matrices:
            g = self.engine.groups[m.group_idx]
            if m.owner != g.dp_rank:
                m.momentum = None
                continue
            t = sd.get(m.key)
            if t is None:      # files written before keys became layout independent
                t = sd.get(f"{m.slot.name}|{m.expert}|{m.col_lo}")
            if t is not None and tuple(t.shape) == tuple(m.full_shape):
                m.momentum = t.to(g.device).float().clone()
