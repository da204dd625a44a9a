"""Flat-buffer optimizer engine: DP gradient reduction, TP-aware global-norm clipping,
fused Adam and ZeRO-1 optimizer-state sharding.

Layout. Parameters are re-pointed into one contiguous buffer per reduction group (dense
parameters reduce over the data-parallel group, expert parameters over the
expert-data-parallel group). Inside a buffer, parameters are ordered into regions
``[TP-sharded | TP-replicated] x [decay | no-decay | muon]`` so that every per-region
operation (squared norm, Adam with one weight-decay value, the TP all-reduce that
sequence parallelism needs for replicated parameters) is a single contiguous range.
Gradients accumulate in a flat ``main_grad`` buffer (fp32 by default): linear layers
add ``x^T dy`` into it from the GEMM epilogue, every other parameter through a
post-accumulate hook.

Step (ZeRO-1): reduce-scatter grads over DP -> squared-norm of the local shard ->
scalar all-reduce -> clip coefficient (device) -> Adam on the shard (moments exist only
for the shard) -> all-gather parameters. With ``zero_stage = 0`` the reduce-scatter /
all-gather pair becomes one all-reduce and every rank updates everything.
The update rule is the reference's (see :mod:`ironcore_b200.optim.adam`).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import kernels
from ..parallel import mesh
from .adam import adam_update_reference

_ALIGN = 64  # elements; keeps every parameter 128-byte aligned for TMA


def _gsize(group) -> int:
    return dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1


def _grank(group) -> int:
    return dist.get_rank(group) if (group is not None and dist.is_initialized()) else 0


def is_no_decay(module: nn.Module, param_name: str, no_decay_on_embedding: bool) -> bool:
    """bias, norm gains, and (optionally) learned position tables are not decayed; word
    embeddings are. (Behavioural reference: ironcore/optimizer/__init__.py:33-52.)"""
    from ..layers.norm import _NormParams

    if param_name.endswith("bias"):
        return True
    if isinstance(module, (_NormParams, nn.LayerNorm, nn.RMSNorm)):
        return True
    if isinstance(module, nn.Embedding) and param_name == "weight":
        return bool(no_decay_on_embedding)
    return False


def is_muon_param(name: str, p: torch.Tensor) -> bool:
    """2-D hidden weight matrices (attention and MLP projections, expert matrices); not
    embeddings, LM head, norm gains or biases."""
    if p.dim() < 2 or name.endswith("bias"):
        return False
    if "embedding" in name or "output_layer" in name or "layernorm" in name or "router" in name:
        return False
    return True


def muon_param_group(o) -> dict:
    """Param group of the Muon matrices. The schedule is computed on the Adam scale (``initial_lr`` =
    ``max_lr``, floor ``min_lr``) and multiplied by ``lr_mult = muon_lr / max_lr`` exactly once, so the
    Muon rate follows the same warm-up / decay shape and peaks at ``muon_lr``."""
    mult = o.muon_lr / o.max_lr if o.max_lr else 1.0
    base = o.max_lr if o.max_lr else o.muon_lr
    return {"lr": o.muon_lr, "initial_lr": base, "name": "muon", "lr_mult": mult}


@dataclass
class Region:
    start: int
    end: int
    weight_decay: float
    tp_replicated: bool
    kind: str  # "adam" | "muon"


@dataclass
class Slot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    region: int


class FlatGroup:
    """One contiguous parameter buffer + gradient buffer reduced over ``group``."""

    def __init__(self, named_params, reduce_group, weight_decay: float, decay_fn, muon_fn, grad_dtype, pad_to: int,
                 alloc=None):
        self.reduce_group = reduce_group
        self.dp = _gsize(reduce_group)
        self.dp_rank = _grank(reduce_group)
        buckets: Dict[tuple, list] = {}
        order = []
        for name, mod, pname, p in named_params:
            # not sharded over the tensor-parallel group: every TP rank holds a copy (norms, biases of row-parallel
            # layers, the router, and the expert weights, which are split over the expert-parallel group only)
            repl = getattr(p, "tp_shard_dim", None) is None
            kind = "muon" if muon_fn(name, p) else "adam"
            wd = 0.0 if decay_fn(mod, pname) else weight_decay
            key = (repl, kind, wd)
            if key not in buckets:
                buckets[key] = []
                order.append(key)
            buckets[key].append((name, p))
        order.sort(key=lambda k: (k[0], k[1] != "adam", k[2] == 0.0))
        self.slots: List[Slot] = []
        self.regions: List[Region] = []
        off = 0
        for key in order:
            start = off
            for name, p in buckets[key]:
                n = p.numel()
                self.slots.append(Slot(name, p, off, n, len(self.regions)))
                off += (n + _ALIGN - 1) // _ALIGN * _ALIGN
            self.regions.append(Region(start, off, key[2], key[0], key[1]))
        unit = max(pad_to * self.dp, _ALIGN)
        self.total = (off + unit - 1) // unit * unit if off > 0 else 0
        first = self.slots[0].param if self.slots else None
        self.dtype = first.dtype if first is not None else torch.float32
        self.device = first.device if first is not None else torch.device("cpu")
        # ``alloc(group, param_dtype, grad_dtype)`` may place both buffers in symmetric memory (fused ZeRO step)
        bufs = alloc(self, self.dtype, grad_dtype or self.dtype) if (alloc is not None and self.total > 0) else None
        if bufs is not None:
            self.param_buf, self.grad_buf = bufs
        else:
            self.param_buf = torch.zeros(self.total, dtype=self.dtype, device=self.device)
            self.grad_buf = torch.zeros(self.total, dtype=grad_dtype or self.dtype, device=self.device)
        for s in self.slots:
            view = self.param_buf[s.offset:s.offset + s.numel].view(s.param.shape)
            view.copy_(s.param.data)
            s.param.data = view
            s.param.main_grad = self.grad_buf[s.offset:s.offset + s.numel].view(s.param.shape)
            s.param.grad_ready = False
        self.shard_size = self.total // self.dp if self.dp > 0 else self.total
        self.buckets: List[Tuple[int, int, int]] = []   # (start, end, number of slots) of every reduction bucket
        self.slot_bucket: List[int] = []                 # bucket of slot i

    def make_buckets(self, bucket_elems: int) -> None:
        """Cut the flat buffer into contiguous ranges of about ``bucket_elems`` elements that begin and end on
        parameter boundaries (the last one takes the padding at the end of the buffer)."""
        self.buckets, self.slot_bucket = [], []
        start, count = 0, 0
        for i, s in enumerate(self.slots):
            self.slot_bucket.append(len(self.buckets))
            count += 1
            end = self.slots[i + 1].offset if i + 1 < len(self.slots) else self.total
            if end - start >= bucket_elems or i + 1 == len(self.slots):
                self.buckets.append((start, end, count))
                start, count = end, 0

    def shard_range(self, sharded: bool):
        if not sharded:
            return 0, self.total
        return self.dp_rank * self.shard_size, (self.dp_rank + 1) * self.shard_size


class DistributedOptimizer:
    """Adam (and hooks for Muon) over flat buffers with optional ZeRO-1 sharding."""

    def __init__(self, model: nn.Module, config, dp_group="default", edp_group="default", tp_group="default",
                 muon=None):
        o = config.optim
        self.config = config
        self.dp_group = mesh.get_data_parallel_group() if dp_group == "default" else dp_group
        self.edp_group = mesh.get_expert_data_parallel_group() if edp_group == "default" else edp_group
        self.tp_group = mesh.get_tensor_model_parallel_group() if tp_group == "default" else tp_group
        self.tp_size = _gsize(self.tp_group)
        # every gradient (dense or expert) is a sum over all data-parallel ranks' losses once its
        # reduction group has been summed (expert gradients already contain the tokens of the
        # whole EP group), so the mean divides by the full data-parallel size
        self.grad_div = float(_gsize(self.dp_group))
        self.sequence_parallel = mesh.sequence_parallel_enabled()
        self.zero = int(config.parallel.zero_stage) >= 1
        self.lr = o.max_lr
        self.betas = (o.adam_beta1, o.adam_beta2)
        self.eps = o.adam_eps
        self.clip = float(o.clip_grad or 0.0)
        self.offload = bool(o.cpu_offload_optimizer)
        self.use_muon = o.optimizer.lower() == "muon"
        self.step_count = 0
        grad_dtype = torch.float32 if getattr(o, "fp32_grad_accum", True) else None
        self.model = model
        named = []
        for mn, mod in model.named_modules():
            for pn, p in mod.named_parameters(recurse=False):
                if not p.requires_grad:
                    continue
                named.append((f"{mn}.{pn}" if mn else pn, mod, pn, p))
        seen = set()
        uniq = []
        for item in named:
            if id(item[3]) in seen:
                continue
            seen.add(id(item[3]))
            uniq.append(item)
        decay_fn = lambda mod, pn: is_no_decay(mod, pn, o.no_decay_on_embedding)
        muon_fn = (lambda n, p: is_muon_param(n, p)) if self.use_muon else (lambda n, p: False)
        dense = [it for it in uniq if not getattr(it[3], "expert_parallel", False)]
        expert = [it for it in uniq if getattr(it[3], "expert_parallel", False)]
        self.groups: List[FlatGroup] = []
        self.fused_zero = None
        alloc = None
        if self.zero and not expert and not self.use_muon and not self.offload and self.tp_size == 1 \
                and _gsize(self.dp_group) > 1 and getattr(config.parallel, "fused_comm", True) \
                and grad_dtype == torch.float32 and dense and dense[0][3].is_cuda \
                and dense[0][3].dtype in (torch.bfloat16, torch.float16) \
                and not getattr(config.parallel, "overlap_grad_reduce", False):
            from .fused_zero import FusedZeroStep

            self.fused_zero = FusedZeroStep.create(self.dp_group)
            alloc = self.fused_zero.allocate if self.fused_zero is not None else None
        if dense:
            self.groups.append(FlatGroup(dense, self.dp_group, o.weight_decay, decay_fn, muon_fn, grad_dtype, 128,
                                         alloc=alloc))
        if expert:
            self.groups.append(FlatGroup(expert, self.edp_group, o.weight_decay, decay_fn, muon_fn, grad_dtype, 128))
        self.param_groups = [{"lr": o.max_lr, "initial_lr": o.max_lr, "name": "adam"}]
        if self.use_muon:
            self.param_groups.append(muon_param_group(o))
        # optimizer state: fp32 moments for the adam regions of the local shard
        self.moments = []
        for g in self.groups:
            lo, hi = g.shard_range(self.zero)
            n = hi - lo
            dev = torch.device("cpu") if self.offload else g.device
            kw = dict(dtype=torch.float32, device=dev)
            if self.offload and torch.cuda.is_available():
                kw["pin_memory"] = True
            self.moments.append({"exp_avg": torch.zeros(n, **kw), "exp_avg_sq": torch.zeros(n, **kw)})
        # Overlapped reduction: during the last micro-batch of a step every bucket of the gradient buffer is
        # all-reduced (asynchronously, on the collective library's own stream) as soon as the last of its
        # parameters has its gradient; the step waits for the buckets instead of reducing the whole buffer.
        # (Reference: the bucketed all-reduce of DistributedDataParallel, ironcore/parallel/parallel.py:76-81.)
        self.overlap = bool(getattr(config.parallel, "overlap_grad_reduce", False)) and self.fused_zero is None
        self._overlap_active = False
        self._bucket_left: List[List[int]] = []
        self._bucket_work = []
        if self.overlap:
            for g in self.groups:
                esize = g.grad_buf.element_size() if g.total > 0 else 4
                g.make_buckets(max(int(float(config.parallel.grad_bucket_mb) * (1 << 20)) // esize, 1))
        self._hooks = []
        for gi, g in enumerate(self.groups):
            for si, s in enumerate(g.slots):
                bi = g.slot_bucket[si] if self.overlap and g.dp > 1 else -1
                self._hooks.append(s.param.register_post_accumulate_grad_hook(self._make_hook(gi, bi)))
        self.muon = muon
        if self.use_muon and self.muon is None:
            from .muon import MuonState

            self.muon = MuonState(self, config)
        self._norm = None
        self._side_stream = None

    def _make_hook(self, group_index: int, bucket_index: int):
        def hook(p):
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None
            if bucket_index >= 0 and self._overlap_active:
                left = self._bucket_left[group_index]
                left[bucket_index] -= 1
                if left[bucket_index] == 0:
                    self._launch_bucket(group_index, bucket_index)
        return hook

    def _launch_bucket(self, group_index: int, bucket_index: int):
        g = self.groups[group_index]
        a, b, _ = g.buckets[bucket_index]
        self._bucket_left[group_index][bucket_index] = -1     # launched
        if b > a:
            self._bucket_work.append(dist.all_reduce(g.grad_buf[a:b], group=g.reduce_group, async_op=True))

    def start_grad_reduce_overlap(self) -> bool:
        """Call before the backward pass of the step's last micro-batch. Returns whether buckets will be reduced
        behind that pass (``parallel.overlap_grad_reduce`` and a data-parallel group of more than one rank)."""
        if not self.overlap or not any(g.dp > 1 for g in self.groups):
            return False
        self._bucket_left = [[n for _, _, n in g.buckets] if g.dp > 1 else [] for g in self.groups]
        self._bucket_work = []
        self._overlap_active = True
        return True

    def _finish_grad_reduce_overlap(self):
        """Reduce the buckets whose parameters received no gradient in the last micro-batch, then wait for all."""
        self._overlap_active = False
        for gi, left in enumerate(self._bucket_left):
            for bi, n in enumerate(left):
                if n >= 0:
                    self._launch_bucket(gi, bi)
        for w in self._bucket_work:
            w.wait()
        self._bucket_work = []

    # ------------------------------------------------------------------ API
    def zero_grad(self, set_to_none: bool = False):
        for g in self.groups:
            g.grad_buf.zero_()
            for s in g.slots:
                s.param.grad = None

    @property
    def grad_norm(self):
        return self._norm

    def _tp_sync_replicated(self, g: FlatGroup):
        """Sequence parallelism: TP-replicated parameters saw different tokens on every TP
        rank, so their gradients are summed over the TP group."""
        if not (self.sequence_parallel and self.tp_size > 1):
            return
        for r in g.regions:
            if r.tp_replicated and r.end > r.start:
                dist.all_reduce(g.grad_buf[r.start:r.end], group=self.tp_group)

    def _reduce_grads(self, g: FlatGroup):
        if g.dp == 1:
            return
        if self.zero:
            lo, hi = g.shard_range(True)
            # Muon owners need the whole gradient of their matrices, which lie outside their Adam shard:
            # with Muon the buffer is all-reduced (the optimizer state stays sharded either way).
            if g.device.type == "cpu" or self.use_muon:
                dist.all_reduce(g.grad_buf, group=g.reduce_group)
            else:
                dist.reduce_scatter_tensor(g.grad_buf[lo:hi], g.grad_buf, group=g.reduce_group)
        else:
            dist.all_reduce(g.grad_buf, group=g.reduce_group)

    def _sumsq(self, buf: torch.Tensor, out: torch.Tensor, weight: float):
        if buf.numel() == 0:
            return
        if buf.is_cuda:
            tmp = torch.zeros(1, dtype=torch.float32, device=buf.device)
            kernels.sumsq(buf, tmp)
            out.add_(tmp * weight)
        else:
            out.add_(buf.float().pow(2).sum() * weight)

    def _global_norm_and_coef(self):
        """Returns (norm, coef) device tensors. Gradients hold sums over DP ranks; the true
        gradient is sum / dp, which is folded into the returned norm and into Adam's scale."""
        dev = self.groups[0].device if self.groups else torch.device("cpu")
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        for g in self.groups:
            lo, hi = g.shard_range(self.zero)
            inv = 1.0 / (self.grad_div * self.grad_div)
            for r in g.regions:
                a, b = max(r.start, lo), min(r.end, hi)
                if b <= a:
                    continue
                w = inv / self.tp_size if r.tp_replicated else inv
                self._sumsq(g.grad_buf[a:b], total, w)
        if dist.is_initialized() and mesh.get_world_size() > 1:
            # sharded regions: sum over TP; ZeRO shards: sum over DP. Replicated regions were
            # pre-divided by tp. Every rank of the world contributes exactly its own part when
            # ZeRO is on; otherwise DP replicas hold identical values, so only reduce over TP
            # (and over EP for expert shards, which differ per EP rank).
            if self.zero:
                dist.all_reduce(total, group=None)
                # dense (non-expert) ranges are partitioned across DP; expert ranges across EDP but
                # differ per EP rank, so a world-wide sum counts everything exactly once.
            else:
                if self.tp_size > 1:
                    dist.all_reduce(total, group=self.tp_group)
                ep_group = mesh.get_expert_model_parallel_group()
                if len(self.groups) > 1 and _gsize(ep_group) > 1:
                    # expert shards differ across EP ranks: add the other ranks' expert parts
                    dense_total = torch.zeros_like(total)
                    g0 = self.groups[0]
                    inv0 = 1.0 / (self.grad_div * self.grad_div)
                    for r in g0.regions:
                        w = inv0 / self.tp_size if r.tp_replicated else inv0
                        self._sumsq(g0.grad_buf[r.start:r.end], dense_total, w)
                    if self.tp_size > 1:
                        dist.all_reduce(dense_total, group=self.tp_group)
                    expert_total = total - dense_total
                    dist.all_reduce(expert_total, group=ep_group)
                    total = dense_total + expert_total
        if total.is_cuda:
            norm, coef = kernels.clip_coef(total, self.clip)
        else:
            norm = total.sqrt()
            coef = torch.clamp(self.clip / (norm + 1e-6), max=1.0) if self.clip > 0 else torch.ones_like(norm)
        return norm, coef

    @torch.no_grad()
    def param_norm(self) -> torch.Tensor:
        """L2 norm of all parameters of the model (not only this rank's): one sum-of-squares kernel per
        region of the flat parameter buffer instead of a loop over tensors; regions replicated over the
        tensor-parallel group are counted once, sharded ones are summed over TP (and expert regions over
        the expert-parallel group). (Reference: the per-parameter loop of ironcore/trainer.py:335-340.)"""
        dev = self.groups[0].device if self.groups else torch.device("cpu")
        dense = torch.zeros(1, dtype=torch.float32, device=dev)
        expert = torch.zeros(1, dtype=torch.float32, device=dev)
        for gi, g in enumerate(self.groups):
            is_expert = gi > 0
            for r in g.regions:
                if r.end <= r.start:
                    continue
                w = 1.0 / self.tp_size if r.tp_replicated and not is_expert else 1.0
                self._sumsq(g.param_buf[r.start:r.end], expert if is_expert else dense, w)
        if dist.is_initialized():
            if self.tp_size > 1:
                dist.all_reduce(dense, group=self.tp_group)
            ep_group = mesh.get_expert_model_parallel_group()
            if len(self.groups) > 1 and _gsize(ep_group) > 1:
                dist.all_reduce(expert, group=ep_group)
        return (dense + expert).sqrt().squeeze(0)

    def _adam_range(self, g: FlatGroup, mom, lo: int, a: int, b: int, wd: float, coef, lr: float):
        """Adam on flat range [a, b) of group g; moments are indexed relative to ``lo``."""
        p = g.param_buf[a:b]
        gr = g.grad_buf[a:b]
        b1, b2 = self.betas
        gscale = 1.0 / self.grad_div
        if self.offload:
            self._adam_offloaded(p, gr, mom, a - lo, b - lo, wd, coef, lr, gscale)
            return
        m = mom["exp_avg"][a - lo:b - lo]
        v = mom["exp_avg_sq"][a - lo:b - lo]
        if p.is_cuda:
            kernels.adam_step_(p, gr, m, v, lr=lr, beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd,
                               step=self.step_count, grad_scale=gscale, grad_scale_dev=coef)
        else:
            adam_update_reference(p, gr, m, v, lr=lr, beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd,
                                  step=self.step_count, grad_scale=gscale * float(coef))

    def _adam_offloaded(self, p, gr, mom, a, b, wd, coef, lr, gscale, chunk: int = 1 << 24):
        """Moments live in pinned host memory: stream them through the device in chunks on a
        side stream (H2D, update, D2H), double-buffered against the main stream's work."""
        b1, b2 = self.betas
        if not p.is_cuda:
            adam_update_reference(p, gr, mom["exp_avg"][a:b], mom["exp_avg_sq"][a:b], lr=lr, beta1=b1, beta2=b2,
                                  eps=self.eps, weight_decay=wd, step=self.step_count,
                                  grad_scale=gscale * float(coef))
            return
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream()
        side = self._side_stream
        side.wait_stream(torch.cuda.current_stream())
        n = b - a
        with torch.cuda.stream(side):
            for c0 in range(0, n, chunk):
                c1 = min(n, c0 + chunk)
                hm = mom["exp_avg"][a + c0:a + c1]
                hv = mom["exp_avg_sq"][a + c0:a + c1]
                dm = hm.to(p.device, non_blocking=True)
                dv = hv.to(p.device, non_blocking=True)
                kernels.adam_step_(p[c0:c1], gr[c0:c1], dm, dv, lr=lr, beta1=b1, beta2=b2, eps=self.eps,
                                   weight_decay=wd, step=self.step_count, grad_scale=gscale, grad_scale_dev=coef)
                hm.copy_(dm, non_blocking=True)
                hv.copy_(dv, non_blocking=True)
        # step() joins the side stream after the Muon matrices were updated on the main stream: the
        # host <-> device traffic of the moments overlaps the Newton-Schulz GEMMs (disjoint parameters)
        self._side_pending = True

    def _fused_zero_step(self):
        """Gradient reduce-scatter, global norm, Adam and parameter all-gather in two kernels that talk
        to the peers' buffers directly (pure data parallelism, one flat group)."""
        g, mom = self.groups[0], self.moments[0]
        lo, hi = g.shard_range(True)
        inv = 1.0 / (self.grad_div * self.grad_div)
        regions = []
        for r in g.regions:
            a, b = max(r.start, lo), min(r.end, hi)
            if b > a:
                regions.append((a, b, inv, r.weight_decay, 1.0 if r.kind == "adam" else 0.0))
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        lr = self.param_groups[0]["lr"]
        return self.fused_zero.step(regions, lo, mom["exp_avg"], mom["exp_avg_sq"], lr=lr, beta1=b1, beta2=b2,
                                    eps=self.eps, step_size=lr * (bc2 ** 0.5) / bc1, grad_scale=1.0 / self.grad_div,
                                    clip=self.clip)

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        if self.fused_zero is not None and self.fused_zero.ready:
            self._norm = self._fused_zero_step()
            return self._norm
        overlapped = self._overlap_active
        if overlapped:
            self._finish_grad_reduce_overlap()
        for g in self.groups:
            self._tp_sync_replicated(g)
            if not (overlapped and g.dp > 1):
                self._reduce_grads(g)
        norm, coef = self._global_norm_and_coef()
        self._norm = norm
        lr = self.param_groups[0]["lr"]
        for g, mom in zip(self.groups, self.moments):
            lo, hi = g.shard_range(self.zero)
            for r in g.regions:
                if r.kind != "adam":
                    continue
                a, b = max(r.start, lo), min(r.end, hi)
                if b > a:
                    self._adam_range(g, mom, lo, a, b, r.weight_decay, coef, lr)
        if self.use_muon and self.muon is not None:
            self.muon.step(coef, self.param_groups[1]["lr"])
        if getattr(self, "_side_pending", False):
            torch.cuda.current_stream().wait_stream(self._side_stream)
            self._side_pending = False
        if self.zero:
            for g in self.groups:
                if g.dp > 1:
                    lo, hi = g.shard_range(True)
                    if g.device.type == "cpu":
                        parts = [torch.empty(g.shard_size, dtype=g.dtype) for _ in range(g.dp)]
                        dist.all_gather(parts, g.param_buf[lo:hi].clone(), group=g.reduce_group)
                        g.param_buf.copy_(torch.cat(parts))
                    else:
                        dist.all_gather_into_tensor(g.param_buf, g.param_buf[lo:hi].clone(), group=g.reduce_group)
        return norm

    # ------------------------------------------------------------------ checkpoint state
    def state_dict(self) -> dict:
        """Per-parameter-name state ``{step, exp_avg, exp_avg_sq}`` (full tensors: ZeRO shards
        are gathered over the reduction group), plus param_groups."""
        state = {}
        for g, mom in zip(self.groups, self.moments):
            full = {}
            for key in ("exp_avg", "exp_avg_sq"):
                t = mom[key]
                if self.zero and g.dp > 1:
                    loc = t.to(g.device)
                    if g.device.type == "cpu":
                        parts = [torch.empty_like(loc) for _ in range(g.dp)]
                        dist.all_gather(parts, loc, group=g.reduce_group)
                        t = torch.cat(parts)
                    else:
                        out = torch.empty(g.total, dtype=torch.float32, device=g.device)
                        dist.all_gather_into_tensor(out, loc.contiguous(), group=g.reduce_group)
                        t = out
                full[key] = t
            for s in g.slots:
                if g.regions[s.region].kind != "adam":
                    continue
                state[s.name] = {
                    "step": self.step_count,
                    "exp_avg": full["exp_avg"][s.offset:s.offset + s.numel].view(s.param.shape).clone().cpu(),
                    "exp_avg_sq": full["exp_avg_sq"][s.offset:s.offset + s.numel].view(s.param.shape).clone().cpu(),
                }
        out = {"state": state, "param_groups": [dict(pg) for pg in self.param_groups], "step": self.step_count}
        if self.use_muon and self.muon is not None:
            out["muon"] = self.muon.state_dict()
        return out

    def load_state_dict(self, sd: dict):
        self.step_count = int(sd.get("step", 0))
        for pg, saved in zip(self.param_groups, sd.get("param_groups", [])):
            pg.update({k: v for k, v in saved.items() if k in ("lr", "initial_lr")})
        state = sd.get("state", {})
        for g, mom in zip(self.groups, self.moments):
            lo, hi = g.shard_range(self.zero)
            for s in g.slots:
                st = state.get(s.name)
                if st is None:
                    continue
                self.step_count = max(self.step_count, int(st.get("step", 0)))
                for key in ("exp_avg", "exp_avg_sq"):
                    src = st[key].reshape(-1).float()
                    a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
                    if b > a:
                        mom[key][a - lo:b - lo].copy_(src[a - s.offset:b - s.offset])
        if self.use_muon and self.muon is not None and "muon" in sd:
            self.muon.load_state_dict(sd["muon"])
        return self
