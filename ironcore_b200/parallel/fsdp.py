"""Fully sharded data parallelism (ZeRO-3 style) over the data-parallel group.

Units. The embedding / final norm / LM head form one unit and every transformer layer is a
unit. A unit's parameters live in one flat buffer; each rank keeps only ``1/dp`` of it (the
shard, optionally in pinned host memory with ``fsdp_offload_params``). Before a unit runs
(forward, and again before its backward) the full buffer is re-materialised by an
all-gather into storage that is resized in place, so the parameter tensors — views of that
storage — stay valid for autograd; afterwards the storage is shrunk to zero. The next unit's
all-gather is prefetched on a communication stream. When all gradients of a unit have been
produced they are packed into a flat buffer and reduce-scattered (in fp32 for ``mixed`` /
``fp32`` precision, else in the parameter dtype) into the rank's fp32 gradient shard, which
accumulates over micro-batches.

Optimizer. Adam runs on the shard ranges (decay / no-decay split); the global gradient norm is
the all-reduced sum of shard norms; with ``optim.cpu_offload_optimizer`` the Adam moments live in
pinned host memory and stream through the device on a side stream while the Muon matrices are
updated. With Muon every logical matrix has an owner rank: each rank sends the pieces of its
gradient shard to the owners of the matrices they belong to (one all-to-all of 4 bytes per local
Muon parameter), the owner runs Newton-Schulz on the assembled matrix and returns the update pieces
in the parameter dtype to the shard holders (a second all-to-all of 2 bytes per parameter) —
momentum, orthogonalisation work and wire bytes are all divided by ``dp``.
Strategies: ``full`` (default), ``hybrid`` (same as full inside one node) and ``no_shard``
(parameters stay whole; gradients are all-reduced).
(The reference's FSDP branch — ironcore/parallel/parallel.py:82-115 — never shards anything;
the configuration names are kept.)
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import kernels
from ..optim.adam import adam_update_reference
from ..optim.distributed import is_muon_param, is_no_decay, muon_param_group
from . import mesh

_ALIGN = 64


def _gsize(g):
    return dist.get_world_size(g) if (g is not None and dist.is_initialized()) else 1


def _grank(g):
    return dist.get_rank(g) if (g is not None and dist.is_initialized()) else 0


class FSDPUnit:
    def __init__(self, name: str, named_params, group, weight_decay: float, no_decay_on_embedding: bool,
                 use_muon: bool, reduce_dtype, shard: bool, offload: bool, offload_state: bool = False):
        self.name = name
        self.group = group
        self.dp, self.rank = _gsize(group), _grank(group)
        self.shard_params = shard and self.dp > 1
        self.reduce_dtype = reduce_dtype
        # order: adam+decay | adam+no-decay | muon
        def key(item):
            n, mod, pn, p = item
            muon = use_muon and is_muon_param(n, p)
            nd = is_no_decay(mod, pn, no_decay_on_embedding)
            return (2 if muon else (1 if nd else 0))

        items = sorted(named_params, key=key)
        self.params: List[nn.Parameter] = []
        self.names: List[str] = []
        self.offsets: List[int] = []
        self.kinds: List[int] = []
        off = 0
        for it in items:
            n, mod, pn, p = it
            self.names.append(n)
            self.params.append(p)
            self.offsets.append(off)
            self.kinds.append(key(it))
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.bounds = [0, 0, 0, off]  # start of kind 0, 1, 2 and end
        for k in (1, 2):
            idx = [i for i, kk in enumerate(self.kinds) if kk >= k]
            self.bounds[k] = self.offsets[idx[0]] if idx else off
        unit = _ALIGN * self.dp
        self.total = (off + unit - 1) // unit * unit
        self.shard_size = self.total // self.dp
        p0 = self.params[0]
        self.dtype, self.device = p0.dtype, p0.device
        self.weight_decay = weight_decay
        full = torch.zeros(self.total, dtype=self.dtype, device=self.device)
        for p, o in zip(self.params, self.offsets):
            full[o:o + p.numel()].copy_(p.data.reshape(-1))
        self.full = full
        lo = self.rank * self.shard_size
        self.shard = full[lo:lo + self.shard_size].clone() if self.shard_params else None
        self.offload = offload and self.shard_params and self.device.type == "cuda"
        if self.offload:
            self.shard_host = self.shard.cpu().pin_memory()
            self.shard = None
        for p, o in zip(self.params, self.offsets):
            p.data = full[o:o + p.numel()].view(p.shape)
        self.materialised = True
        self.grad_shard = torch.zeros(self.shard_size if self.shard_params else self.total, dtype=torch.float32,
                                      device=self.device)
        # Adam moments: on the device, or (``optim.cpu_offload_optimizer``) in pinned host memory
        self.offload_state = bool(offload_state) and self.device.type == "cuda"
        if self.offload_state:
            self.exp_avg = torch.zeros(self.grad_shard.shape, dtype=torch.float32).pin_memory()
            self.exp_avg_sq = torch.zeros(self.grad_shard.shape, dtype=torch.float32).pin_memory()
        else:
            self.exp_avg = torch.zeros_like(self.grad_shard)
            self.exp_avg_sq = torch.zeros_like(self.grad_shard)
        self._flat_grad: Optional[torch.Tensor] = None
        self._pending = 0
        self.gather_event = None
        # in-kernel parameter gather (``parallel.fsdp_fused_gather``): set by ``FullyShardedModel``
        self.pool = None            # FsdpCommPool shared by all units
        self.pool_slot = 0          # this unit's slot: fixed, so its parameters always live at the same address
        self.pool_stream = None     # stream the gather kernels run on
        self.use_pool = False
        self._pool_full: Optional[torch.Tensor] = None
        self._points_at = full.data_ptr()
        if self.shard_params:
            self.release()

    # ---- parameter materialisation ----
    def _local_shard(self) -> torch.Tensor:
        if self.offload:
            return self.shard_host.to(self.device, non_blocking=True)
        return self.shard

    def _point_params(self, buf: torch.Tensor):
        if self._points_at == buf.data_ptr():
            return
        for p, o in zip(self.params, self.offsets):
            p.data = buf[o:o + p.numel()].view(p.shape)
        self._points_at = buf.data_ptr()

    def _gather_in_kernel(self, async_op: bool):
        """Gather into this unit's slot of the symmetric pool with the P2P / multicast kernel, on the pool's
        stream. The kernel starts once everything the compute stream has been given so far is done (the slot's
        previous tenant included) and runs beside what the compute stream is given next."""
        comm = self.pool_stream
        comm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(comm):
            shard = self._local_shard()
            full = self.pool.gather(shard, self.pool_slot)
            event = torch.cuda.Event()
            event.record(comm)
        self._gather_event = event
        self._gather_src = shard
        self._pool_full = full
        self._point_params(full)
        self.materialised = True
        if not async_op:
            self.wait_gather()

    def gather(self, async_op: bool = False):
        """Re-materialise the full buffer. With ``async_op`` the all-gather is only enqueued (it runs on the
        communication stream of the backend, overlapping whatever the compute stream does next); ``wait_gather``
        makes the compute stream wait for it right before the unit's parameters are used."""
        if self.materialised or not self.shard_params:
            return
        if self.use_pool and self.pool is not None:
            self._gather_in_kernel(async_op)
            return
        nbytes = self.total * self.full.element_size()
        self.full.untyped_storage().resize_(nbytes)
        if self.pool is not None:
            self._point_params(self.full)     # the parameters may still be views of a pool slot
        shard = self._local_shard()
        if self.device.type == "cpu":
            parts = [torch.empty_like(shard) for _ in range(self.dp)]
            dist.all_gather(parts, shard, group=self.group)
            self.full.copy_(torch.cat(parts))
        else:
            work = dist.all_gather_into_tensor(self.full, shard, group=self.group, async_op=async_op)
            self._gather_work = work if async_op else None
            self._gather_src = shard if async_op else None   # keep the source alive until the wait
        self.materialised = True

    def wait_gather(self):
        event = getattr(self, "_gather_event", None)
        if event is not None:
            torch.cuda.current_stream().wait_event(event)
            self._gather_event = None
            self._gather_src = None
        work = getattr(self, "_gather_work", None)
        if work is not None:
            work.wait()
            self._gather_work = None
            self._gather_src = None

    def release(self):
        if not self.shard_params or not self.materialised:
            return
        self.wait_gather()
        if self._pool_full is not None:
            # the slot keeps the bytes until its next tenant's gather, which waits for this stream first
            self._pool_full = None
        else:
            self.full.untyped_storage().resize_(0)
        self.materialised = False

    def write_back_shard(self, new_shard: torch.Tensor):
        if self.offload:
            self.shard_host.copy_(new_shard, non_blocking=True)
        elif self.shard is not new_shard:
            self.shard.copy_(new_shard)

    # ---- gradients ----
    def begin_backward(self):
        self._pending = sum(1 for p in self.params if p.requires_grad)
        self._flat_grad = torch.zeros(self.total, dtype=self.reduce_dtype, device=self.device)

    def grad_ready(self, idx: int):
        p = self.params[idx]
        if self._flat_grad is None:
            self.begin_backward()
        o = self.offsets[idx]
        if p.grad is not None:
            self._flat_grad[o:o + p.numel()].copy_(p.grad.reshape(-1))
            p.grad = None
        self._pending -= 1
        if self._pending == 0:
            self.reduce_grads()

    def reduce_grads(self):
        fg = self._flat_grad
        self._flat_grad = None
        if self.dp > 1:
            if self.shard_params:
                out = torch.empty(self.shard_size, dtype=fg.dtype, device=fg.device)
                if self.device.type == "cpu":
                    dist.all_reduce(fg, group=self.group)
                    out.copy_(fg[self.rank * self.shard_size:(self.rank + 1) * self.shard_size])
                    self.grad_shard.add_(out.float())
                else:
                    # enqueue only: the reduce-scatter overlaps the backward pass of the next unit; the sum
                    # is folded into the fp32 shard by ``finish_reduction`` (next unit's reduction / optimizer)
                    self.finish_reduction()   # a reduction of an earlier micro-batch may still be pending
                    work = dist.reduce_scatter_tensor(out, fg, group=self.group, async_op=True)
                    self._pending_rs = (work, out, fg)
            else:
                dist.all_reduce(fg, group=self.group)
                self.grad_shard.add_(fg.float())
        else:
            self.grad_shard.add_(fg.float())
        self.release()

    def finish_reduction(self):
        pending = getattr(self, "_pending_rs", None)
        if pending is not None:
            work, out, _fg = pending
            work.wait()
            self.grad_shard.add_(out.float())
            self._pending_rs = None

    def shard_range(self):
        if self.shard_params:
            return self.rank * self.shard_size, (self.rank + 1) * self.shard_size
        return 0, self.total


class FullyShardedModel(nn.Module):
    is_fsdp_wrapper = True

    def __init__(self, model: nn.Module, config):
        super().__init__()
        self.module = model
        self.config = config
        p = config.parallel
        o = config.optim
        self.group = mesh.get_data_parallel_group()
        self.dp = _gsize(self.group)
        self.use_muon = o.optimizer.lower() == "muon"
        mp = p.fsdp_mixed_precision
        dtype = next(model.parameters()).dtype
        reduce_dtype = torch.float32 if mp in ("mixed", "fp32", "float32") else dtype
        shard = p.fsdp_sharding_strategy != "no_shard"
        self.units: List[FSDPUnit] = []
        self._unit_of_module: Dict[int, FSDPUnit] = {}
        layers = list(model.model.layers) if hasattr(model.model, "layers") else []
        layer_ids = set()
        unit_modules = []
        for i, layer in enumerate(layers):
            unit_modules.append((f"layer{i}", layer))
            for m_ in layer.modules():
                layer_ids.add(id(m_))
        root_named = []
        for mn, mod in model.named_modules():
            if id(mod) in layer_ids:
                continue
            for pn, prm in mod.named_parameters(recurse=False):
                root_named.append((f"{mn}.{pn}" if mn else pn, mod, pn, prm))
        mk = lambda name, named: FSDPUnit(name, named, self.group, o.weight_decay, o.no_decay_on_embedding,
                                          self.use_muon, reduce_dtype, shard, p.fsdp_offload_params,
                                          bool(o.cpu_offload_optimizer))
        self.root_unit = mk("root", root_named)
        self.units.append(self.root_unit)
        for i, (name, layer) in enumerate(unit_modules):
            named = []
            prefix = f"model.layers.{i}"
            for mn, mod in layer.named_modules():
                for pn, prm in mod.named_parameters(recurse=False):
                    full_name = ".".join(x for x in (prefix, mn, pn) if x)
                    named.append((full_name, mod, pn, prm))
            u = mk(name, named)
            self.units.append(u)
            self._unit_of_module[id(layer)] = u
            layer.register_forward_pre_hook(self._pre_forward(len(self.units) - 1))
            layer.register_forward_hook(self._post_forward(len(self.units) - 1))
            layer.register_full_backward_pre_hook(self._pre_backward(len(self.units) - 1))
        for u in self.units:
            for idx, prm in enumerate(u.params):
                if prm.requires_grad:
                    prm.register_post_accumulate_grad_hook(self._grad_hook(u, idx))
        self.comm_stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.pool = None
        if getattr(p, "fsdp_fused_gather", False) and shard and self.dp > 1 and self.comm_stream is not None \
                and self.units[0].device.type == "cuda":
            self._attach_gather_pool(dtype, reduce_dtype)

    def _attach_gather_pool(self, dtype, reduce_dtype):
        """Parameter gathers as P2P / NVSwitch-multicast kernels (``csrc/fsdp_comm.cu``) into three symmetric
        slots: one for the root unit, two that the layers alternate between (a layer's slot is fixed, so its
        parameters keep their addresses from gather to gather)."""
        from .fsdp_comm import FsdpCommPool
        from .symmetric import symmetric_memory_available

        if not symmetric_memory_available() or dtype not in (torch.bfloat16, torch.float16):
            return
        quantum = 8 * self.dp
        biggest = max(u.total for u in self.units)
        biggest = (biggest + quantum - 1) // quantum * quantum
        if any(u.total % quantum for u in self.units):
            return
        self.pool = FsdpCommPool(self.group, biggest, dtype, reduce_dtype, slots=3, flat_slots=0)
        for i, u in enumerate(self.units):
            u.pool, u.pool_stream, u.use_pool = self.pool, self.comm_stream, True
            u.pool_slot = 0 if i == 0 else 1 + (i % 2)

    # ---- hooks ----
    def _prefetch(self, idx: int):
        """Enqueue the next unit's all-gather without waiting for it: it overlaps the current unit's compute."""
        if 0 < idx < len(self.units):
            self.units[idx].gather(async_op=True)

    def _pre_forward(self, idx):
        def hook(_m, _inp):
            u = self.units[idx]
            u.gather()
            u.wait_gather()
            self._prefetch(idx + 1)
        return hook

    def _post_forward(self, idx):
        def hook(_m, _inp, _out):
            # the last layer's backward starts right after the forward: keep it materialised
            if idx == len(self.units) - 1 and torch.is_grad_enabled():
                return
            self.units[idx].release()
        return hook

    def _pre_backward(self, idx):
        def hook(_m, _gout):
            u = self.units[idx]
            u.gather()
            u.wait_gather()
            if u._flat_grad is None:
                u.begin_backward()
            self._prefetch(idx - 1 if idx - 1 >= 1 else -1)
        return hook

    def _grad_hook(self, unit: FSDPUnit, idx: int):
        def hook(_p):
            if unit._pending == 1:
                # this is the unit's last gradient: its reduction is about to be issued, so fold the
                # previous one first (at most one unit-sized reduction buffer stays in flight)
                prev = getattr(self, "_last_reduced", None)
                if prev is not None and prev is not unit:
                    prev.finish_reduction()
                self._last_reduced = unit
            unit.grad_ready(idx)
        return hook

    def finish_reductions(self):
        for u in self.units:
            u.finish_reduction()
        self._last_reduced = None

    # ---- nn.Module surface ----
    def forward(self, *a, **k):
        self.root_unit.gather()
        if self.root_unit._flat_grad is None and torch.is_grad_enabled():
            self.root_unit.begin_backward()
        return self.module(*a, **k)

    def gather_all(self):
        """Every unit materialised at once (state dicts): through private buffers, never the shared slots."""
        for u in self.units:
            if u.use_pool:
                u.release()
                u.use_pool = False
            u.gather()
            u.wait_gather()

    def release_all(self):
        for u in self.units:
            if u is not self.root_unit or u.pool is not None:
                u.release()
            u.use_pool = u.pool is not None

    def canonical_state_dict(self):
        self.gather_all()
        sd = {k: v.detach().clone() for k, v in self.module.canonical_state_dict().items()}
        self.release_all()
        return sd

    def canonical_shard_info(self):
        return self.module.canonical_shard_info()

    def load_canonical_state_dict(self, sd, strict=True):
        self.gather_all()
        out = self.module.load_canonical_state_dict(sd, strict=strict)
        for u in self.units:
            if u.shard_params:
                lo, hi = u.shard_range()
                u.write_back_shard(u.full[lo:hi])
        self.release_all()
        return out

    def build_optimizer(self):
        return FSDPOptimizer(self, self.config)


class FSDPOptimizer:
    """Adam / Muon on the FSDP shards with global-norm clipping."""

    def __init__(self, fsdp: FullyShardedModel, config):
        o = config.optim
        self.fsdp = fsdp
        self.config = config
        self.betas = (o.adam_beta1, o.adam_beta2)
        self.eps = o.adam_eps
        self.clip = float(o.clip_grad or 0.0)
        self.step_count = 0
        self.use_muon = fsdp.use_muon
        self.param_groups = [{"lr": o.max_lr, "initial_lr": o.max_lr, "name": "adam"}]
        if self.use_muon:
            self.param_groups.append(muon_param_group(o))
        self.muon_momentum: Dict[str, torch.Tensor] = {}
        self._side_stream = None
        self._side_pending = False
        self._muon_plans: Dict[str, dict] = {}
        self._norm = None
        self._owners: Dict[str, int] = {}
        # Tensor parallelism next to the shard group: a parameter without a tensor-parallel shard dimension is a
        # copy on every TP rank. Its squares count once in a norm summed over the TP group, and under sequence
        # parallelism (each rank sees its token shard) its gradient is the sum over that group.
        self.tp_group = mesh.get_tensor_model_parallel_group()
        self.tp_size = mesh.get_tensor_model_parallel_world_size()
        self.sequence_parallel = mesh.sequence_parallel_enabled() and self.tp_size > 1
        self._tp_copies: Dict[str, list] = {}
        if self.tp_size > 1:
            if self.use_muon:
                raise NotImplementedError("Muon on FSDP shards needs tensor_model_parallel_size 1 (a matrix is "
                                          "orthogonalised from the shards of one group); use the ZeRO-1 engine "
                                          "for tensor-parallel Muon")
            for u in fsdp.units:
                lo, hi = u.shard_range()
                ranges = []
                for p, o in zip(u.params, u.offsets):
                    if getattr(p, "tp_shard_dim", None) is None:
                        a, b = max(o, lo), min(o + p.numel(), hi)
                        if b > a:
                            if ranges and ranges[-1][1] == a - lo:
                                ranges[-1][1] = b - lo          # adjacent copies: one range
                            else:
                                ranges.append([a - lo, b - lo])
                self._tp_copies[u.name] = ranges
        if self.use_muon:
            load = [0.0] * max(fsdp.dp, 1)
            mats = []
            for u in fsdp.units:
                for n, p, k in zip(u.names, u.params, u.kinds):
                    if k == 2:
                        for key, shape in self._logical_matrices(n, p):
                            r, c = min(shape), max(shape)
                            mats.append((4.0 * r * r * c + 2.0 * r ** 3, key))
            for cost, key in sorted(mats, reverse=True):
                r = min(range(len(load)), key=lambda i: load[i])
                self._owners[key] = r
                load[r] += cost

    @staticmethod
    def _logical_matrices(name, p):
        parts = getattr(p, "tp_parts", 1)
        cols = p.shape[-1]
        sizes = [cols // parts] * parts if isinstance(parts, int) else list(parts)
        experts = range(p.shape[0]) if p.dim() == 3 else [None]
        out = []
        for e in experts:
            lo = 0
            for sz in sizes:
                out.append(((name, e, lo, lo + sz), (p.shape[-2], sz)))
                lo += sz
        return out

    def zero_grad(self, set_to_none: bool = False):
        for u in self.fsdp.units:
            u.grad_shard.zero_()

    @property
    def grad_norm(self):
        return self._norm

    def _unit_sumsq(self, u, t: torch.Tensor, total: torch.Tensor) -> None:
        """Add the squares of ``t`` (this rank's flat range of unit ``u``) to ``total``; ranges that are copies on
        every tensor-parallel rank are weighted 1 / tp, so that the sum over that group counts them once."""
        def add(x, w):
            if x.numel() == 0:
                return
            if x.is_cuda:
                tmp = torch.zeros(1, dtype=torch.float32, device=total.device)
                kernels.sumsq(x, tmp)
                total.add_(tmp * w)
            else:
                total.add_(x.float().pow(2).sum() * w)

        add(t, 1.0)
        for a, b in self._tp_copies.get(u.name, ()):
            add(t[a:b], 1.0 / self.tp_size - 1.0)

    @torch.no_grad()
    def param_norm(self) -> torch.Tensor:
        """L2 norm of all parameters: one sum-of-squares kernel per unit shard, summed over the shard group."""
        fs = self.fsdp
        dev = fs.units[0].device
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        sharded = False
        for u in fs.units:
            t = (u._local_shard() if u.shard_params else u.full)
            sharded = sharded or u.shard_params
            self._unit_sumsq(u, t, total)
        if sharded and fs.dp > 1:
            dist.all_reduce(total, group=fs.group)
        if self.tp_size > 1:
            dist.all_reduce(total, group=self.tp_group)
        return total.sqrt().squeeze(0)

    @torch.no_grad()
    def step(self):
        from ..optim.muon import newton_schulz

        fs = self.fsdp
        fs.finish_reductions()
        self.step_count += 1
        dp = float(max(fs.dp, 1))
        dev = fs.units[0].device
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        for u in fs.units:
            if self.sequence_parallel:
                for a, b in self._tp_copies.get(u.name, ()):
                    dist.all_reduce(u.grad_shard[a:b], group=self.tp_group)
            self._unit_sumsq(u, u.grad_shard, total)
        total = total / (dp * dp)
        if fs.dp > 1 and any(u.shard_params for u in fs.units):
            dist.all_reduce(total, group=fs.group)
        if self.tp_size > 1:
            dist.all_reduce(total, group=self.tp_group)
        norm = total.sqrt()
        coef = torch.clamp(self.clip / (norm + 1e-6), max=1.0) if self.clip > 0 else torch.ones_like(norm)
        self._norm = norm
        lr = self.param_groups[0]["lr"]
        b1, b2 = self.betas
        for u in fs.units:
            lo, hi = u.shard_range()
            if u.shard_params:
                pshard = u._local_shard().clone() if u.offload else u.shard
            else:
                pshard = u.full
            ranges = [(u.bounds[0], u.bounds[1], u.weight_decay), (u.bounds[1], u.bounds[2], 0.0)]
            for a, b, wd in ranges:
                a2, b2_ = max(a, lo), min(b, hi)
                if b2_ <= a2:
                    continue
                sl = slice(a2 - lo, b2_ - lo)
                kw = dict(lr=lr, beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd, step=self.step_count)
                if pshard.is_cuda and u.offload_state:
                    self._adam_offloaded(pshard[sl], u.grad_shard[sl], u.exp_avg[sl], u.exp_avg_sq[sl], coef, dp, kw)
                elif pshard.is_cuda:
                    kernels.adam_step_(pshard[sl], u.grad_shard[sl], u.exp_avg[sl], u.exp_avg_sq[sl], grad_scale=1.0 / dp,
                                       grad_scale_dev=coef, **kw)
                else:
                    adam_update_reference(pshard[sl], u.grad_shard[sl], u.exp_avg[sl], u.exp_avg_sq[sl],
                                          grad_scale=float(coef) / dp, **kw)
            if self.use_muon and u.bounds[3] > u.bounds[2]:
                self._muon_unit(u, pshard, lo, hi, coef, dp, newton_schulz)
            if self._side_pending:
                # the offloaded Adam ranges of this unit ran on the side stream, overlapping its Muon matrices
                torch.cuda.current_stream().wait_stream(self._side_stream)
                self._side_pending = False
            if u.shard_params:
                u.write_back_shard(pshard)
        return norm

    def _adam_offloaded(self, p, g, hm, hv, coef, dp, kw, chunk: int = 1 << 24):
        """Adam on a parameter range whose moments live in pinned host memory: the moments stream through the
        device in chunks on a side stream (H2D, update, D2H); ``step`` joins the stream after the unit's Muon
        matrices, which are disjoint parameters updated on the main stream meanwhile."""
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream()
        side = self._side_stream
        side.wait_stream(torch.cuda.current_stream())
        n = p.numel()
        with torch.cuda.stream(side):
            for c0 in range(0, n, chunk):
                c1 = min(n, c0 + chunk)
                dm = hm[c0:c1].to(p.device, non_blocking=True)
                dv = hv[c0:c1].to(p.device, non_blocking=True)
                kernels.adam_step_(p[c0:c1], g[c0:c1], dm, dv, grad_scale=1.0 / dp, grad_scale_dev=coef, **kw)
                hm[c0:c1].copy_(dm, non_blocking=True)
                hv[c0:c1].copy_(dv, non_blocking=True)
        self._side_pending = True

    def _muon_plan(self, u: FSDPUnit) -> dict:
        """Static exchange plan of a unit. A logical matrix (one expert, one fused part) is a set of rows of the
        flat buffer, each row a contiguous run of ``c1 - c0`` elements, cut wherever a shard boundary falls.
        Elements are ordered by (owner, matrix, row, column), which both sides can compute, so nothing but the
        payload is exchanged.
          send[r]  : pieces of MY shard that belong to matrices owned by rank r      (gradient: me -> r)
          recv[s]  : pieces of rank s's shard that belong to matrices I own          (gradient: s -> me)
        The update travels the same pieces in the opposite direction."""
        plan = self._muon_plans.get(u.name)
        if plan is not None:
            return plan
        dpn, me, ss = u.dp, u.rank, u.shard_size
        dev = u.device
        send_parts = [[] for _ in range(dpn)]     # per owner: indices into my shard (matrix, row, column order)
        recv_parts = [[] for _ in range(dpn)]     # per source: positions in my packed matrices, same order
        mats, mat_base, total = [], [], 0
        for n, p, k, off in zip(u.names, u.params, u.kinds, u.offsets):
            if k != 2:
                continue
            for key, shape in self._logical_matrices(n, p):
                owner = self._owners.get(key, 0)
                _, e, c0, c1 = key
                rows, cols, width = p.shape[-2], p.shape[-1], c1 - c0
                base = off + (e * rows * cols if e is not None else 0) + c0
                flat = (base + torch.arange(rows, device=dev, dtype=torch.long)[:, None] * cols
                        + torch.arange(width, device=dev, dtype=torch.long)[None, :]).reshape(-1)
                holder = torch.div(flat, ss, rounding_mode="floor")
                send_parts[owner].append(flat[holder == me] - me * ss)
                if owner == me:
                    mats.append((key, shape, rows * width))
                    mat_base.append(total)
                    pos = torch.arange(rows * width, device=dev, dtype=torch.long) + total
                    for s_ in range(dpn):
                        recv_parts[s_].append(pos[holder == s_])
                    total += rows * width
        # 32-bit positions: the cached plans of a 13B model hold one index per Muon parameter of the shard, twice
        empty = torch.zeros(0, dtype=torch.int32, device=dev)
        cat = lambda parts: torch.cat([t.to(torch.int32) for t in parts]) if parts else empty
        per_owner = [cat(send_parts[r]) for r in range(dpn)]
        per_source = [cat(recv_parts[s_]) for s_ in range(dpn)]
        send_index, recv_index = cat(per_owner), cat(per_source)
        # gathers only (index_select takes 32-bit indices, the scatter forms do not): the inverse permutation
        # unpacks the receive buffer into the matrices, and a map over the shard's Muon range (padding -> a
        # trailing zero) applies the returned update
        recv_inverse = torch.argsort(recv_index.long()).to(torch.int32) if recv_index.numel() else empty
        a_, b_ = max(u.bounds[2], me * ss), min(u.bounds[3], (me + 1) * ss)
        span = max(0, b_ - a_)
        apply_map = torch.full((span,), send_index.numel(), dtype=torch.int32, device=dev)
        if send_index.numel():
            apply_map[(send_index.long() - (a_ - me * ss))] = torch.arange(send_index.numel(), device=dev, dtype=torch.int32)
        plan = {
            "recv_inverse": recv_inverse, "apply_map": apply_map, "apply_range": (a_ - me * ss, b_ - me * ss),
            "mats": mats, "mat_base": mat_base, "owned_numel": total,
            "send_splits": [int(t.numel()) for t in per_owner],
            "recv_splits": [int(t.numel()) for t in per_source],
            "send_index": send_index,          # gather from my gradient shard -> send buffer (owner-major)
            "recv_index": recv_index,          # packed matrices I own -> return buffer (source-major)
        }
        self._muon_plans[u.name] = plan
        return plan

    def _muon_unit(self, u: FSDPUnit, pshard, lo, hi, coef, dp, newton_schulz):
        from . import collectives as C

        o = self.config.optim
        lr = self.param_groups[1]["lr"]
        sharded = u.shard_params and u.dp > 1
        if not sharded:
            # whole gradients are local: orthogonalise every matrix in place
            for n, p, k, off in zip(u.names, u.params, u.kinds, u.offsets):
                if k != 2:
                    continue
                g = u.grad_shard[off:off + p.numel()].view(p.shape)
                w = pshard[off:off + p.numel()].view(p.shape)
                for key, shape in self._logical_matrices(n, p):
                    _, e, c0, c1 = key
                    gm = (g[e] if e is not None else g)[:, c0:c1] * (coef / dp)
                    x = self._muon_direction(key, gm, o, newton_schulz)
                    scale = math.sqrt(max(1.0, shape[1] / shape[0]))
                    wm = (w[e] if e is not None else w)[:, c0:c1]
                    if o.muon_weight_decay:
                        wm.mul_(1 - lr * o.muon_weight_decay)
                    wm.add_((x * (-lr * scale)).to(wm.dtype))
            return
        plan = self._muon_plan(u)
        # 1. gradient pieces travel to the owners of their matrices (fp32, 4 bytes per local Muon parameter)
        send = u.grad_shard.index_select(0, plan["send_index"])
        got = C.all_to_all_single(send, plan["recv_splits"], plan["send_splits"], u.group)
        packed = got.index_select(0, plan["recv_inverse"])
        # 2. the owner orthogonalises its matrices
        upd = torch.empty(plan["owned_numel"], dtype=pshard.dtype, device=u.device)
        for (key, shape, numel), base in zip(plan["mats"], plan["mat_base"]):
            gm = packed[base:base + numel].view(shape) * (coef / dp)
            x = self._muon_direction(key, gm, o, newton_schulz)
            scale = math.sqrt(max(1.0, shape[1] / shape[0]))
            upd[base:base + numel].copy_((x * (-lr * scale)).reshape(-1))
        # 3. update pieces return to the shard holders in the parameter dtype (2 bytes per parameter)
        back = C.all_to_all_single(upd.index_select(0, plan["recv_index"]), plan["send_splits"], plan["recv_splits"],
                                   u.group)
        a, b = plan["apply_range"]
        if b > a:
            if o.muon_weight_decay:
                pshard[a:b].mul_(1 - lr * o.muon_weight_decay)
            padded = torch.cat([back.to(pshard.dtype), torch.zeros(1, dtype=pshard.dtype, device=u.device)])
            pshard[a:b].add_(padded.index_select(0, plan["apply_map"]))

    def _muon_direction(self, key, gm, o, newton_schulz):
        """Momentum update and Newton-Schulz orthogonalisation of one matrix gradient (fp32 in, fp32 out)."""
        mom = self.muon_momentum.get(key)
        if mom is None:
            mom = torch.zeros_like(gm)
            self.muon_momentum[key] = mom
        mom.mul_(o.muon_momentum).add_(gm)
        direction = gm.add(mom, alpha=o.muon_momentum) if o.nesterov else mom
        return newton_schulz(direction.contiguous(), o.muon_ns_steps).float()

    # ---- checkpoint state (sharded: each rank saves its own moments) ----
    def _full_moment(self, u: FSDPUnit, t: torch.Tensor) -> torch.Tensor:
        if not u.shard_params:
            return t
        if u.device.type == "cpu":
            parts = [torch.empty_like(t) for _ in range(u.dp)]
            dist.all_gather(parts, t, group=u.group)
            return torch.cat(parts)
        out = torch.empty(u.total, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=u.group)
        return out

    def state_dict(self):
        """``fsdp_state_dict_type = full``: per-parameter-name moments gathered over the group
        (collective). Muon momenta are saved by their owners' keys."""
        state = {}
        for u in self.fsdp.units:
            m, v = self._full_moment(u, u.exp_avg), self._full_moment(u, u.exp_avg_sq)
            for n, p, k, off in zip(u.names, u.params, u.kinds, u.offsets):
                if k == 2:
                    continue
                state[n] = {"step": self.step_count,
                            "exp_avg": m[off:off + p.numel()].view(p.shape).clone().cpu(),
                            "exp_avg_sq": v[off:off + p.numel()].view(p.shape).clone().cpu()}
        return {"step": self.step_count, "param_groups": [dict(g) for g in self.param_groups], "state": state,
                "muon": self._muon_state()}

    @staticmethod
    def _muon_key(key) -> str:
        name, e, c0, _ = key
        return f"{name}|{e}|{c0}"

    def _muon_state(self):
        """Momentum of every Muon matrix, broadcast from its owner (collective over the shard group);
        only shard rank 0, the checkpoint writer, keeps the host copies."""
        out = {}
        if not self.use_muon:
            return out
        for u in self.fsdp.units:
            for n, p, k in zip(u.names, u.params, u.kinds):
                if k != 2:
                    continue
                for key, shape in self._logical_matrices(n, p):
                    owner = self._owners.get(key, 0) if (u.dp > 1 and u.shard_params) else u.rank
                    t = self.muon_momentum.get(key) if owner == u.rank else None
                    if u.dp > 1 and u.shard_params:
                        buf = torch.zeros(shape, dtype=torch.float32, device=u.device)
                        if t is not None:
                            buf.copy_(t)
                        dist.broadcast(buf, src=mesh.global_rank_of(u.group, owner), group=u.group)
                        t = buf
                    if t is not None and u.rank == 0:
                        out[self._muon_key(key)] = t.detach().float().cpu()
        return out

    def load_state_dict(self, sd):
        self.step_count = int(sd.get("step", 0))
        state = sd.get("state", {})
        for u in self.fsdp.units:
            lo, hi = u.shard_range()
            for n, p, k, off in zip(u.names, u.params, u.kinds, u.offsets):
                st = state.get(n)
                if st is None or k == 2:
                    continue
                a, b = max(off, lo), min(off + p.numel(), hi)
                if b > a:
                    u.exp_avg[a - lo:b - lo].copy_(st["exp_avg"].reshape(-1)[a - off:b - off])
                    u.exp_avg_sq[a - lo:b - lo].copy_(st["exp_avg_sq"].reshape(-1)[a - off:b - off])
        for pg, saved in zip(self.param_groups, sd.get("param_groups", [])):
            pg.update({k: v for k, v in saved.items() if k in ("lr", "initial_lr")})
        muon = sd.get("muon") or {}
        self.muon_momentum.clear()
        if self.use_muon and muon:
            for u in self.fsdp.units:
                for n, p, k in zip(u.names, u.params, u.kinds):
                    if k != 2:
                        continue
                    for key, shape in self._logical_matrices(n, p):
                        if self._owners.get(key, 0) != u.rank and u.dp > 1 and u.shard_params:
                            continue
                        t = muon.get(self._muon_key(key))
                        if t is not None and tuple(t.shape) == tuple(shape):
                            self.muon_momentum[key] = t.to(u.device).float().clone()
        return self
