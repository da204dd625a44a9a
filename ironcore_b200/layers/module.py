"""Base module: dtype/device properties, weight initialisation and recursive profiler ranges.
(Behavioural reference: ironcore/layers/module.py:19-232.)"""

from __future__ import annotations

import math

import torch
import torch.nn as nn


def init_parameters(module: nn.Module, config, generator: torch.Generator = None) -> None:
    """normal(0, init_std) (or Xavier uniform) for every weight of ``module``; residual projections
    (``attn_output``, ``down_proj``, expert down projections) use std / sqrt(2 * num_layers); biases zero; norm
    gains keep the value set at construction. A sharded weight is this rank's slice of the full tensor, drawn
    from a CPU generator seeded with ``init.seed``, so every tensor-parallel size sees the same full matrices.
    (Behavioural reference: ironcore/layers/module.py:43-163.)"""
    from ..parallel import mesh
    from ..parallel.tensor_parallel import init_linear_weight_

    std = config.init.init_std
    resid_std = std / math.sqrt(2.0 * max(config.model.num_layers, 1))
    gen = generator
    if gen is None:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(int(config.init.seed))
    tp_rank, tp_size = mesh.get_tensor_model_parallel_rank(), mesh.get_tensor_model_parallel_world_size()
    ep_rank = mesh.get_expert_model_parallel_rank()
    ep_size = mesh.get_expert_model_parallel_world_size()
    for name, p in module.named_parameters():
        if name.endswith("bias"):
            nn.init.zeros_(p)
            continue
        if "layernorm" in name:
            continue  # gains were set at construction
        shard_dim = getattr(p, "tp_shard_dim", None)
        parts = getattr(p, "tp_parts", 1)
        is_resid = name.endswith("attn_output.weight") or name.endswith("down_proj.weight") \
            or name.endswith("experts_down")
        s = resid_std if is_resid else std
        if getattr(p, "expert_parallel", False):
            # [E_local, in, out]: draw all experts, keep this rank's slice of the expert dim
            e_local = p.shape[0]
            full = torch.empty((e_local * ep_size,) + tuple(p.shape[1:]), dtype=torch.float32)
            full.normal_(0.0, s, generator=gen)
            with torch.no_grad():
                p.copy_(full[ep_rank * e_local:(ep_rank + 1) * e_local].to(p.dtype))
            continue
        full_shape = list(p.shape)
        if shard_dim is not None and tp_size > 1:
            full_shape[shard_dim] *= tp_size
        if p.dim() < 2:
            with torch.no_grad():
                p.copy_(torch.empty(full_shape).normal_(0.0, s, generator=gen).to(p.dtype))
            continue
        init_linear_weight_(p, full_shape, s, shard_dim, parts, tp_rank, tp_size, bool(config.init.xavier_init), gen,
                            valid=getattr(p, "vocab_valid", None))


class BaseModule(nn.Module):
    def __init__(self, config=None):
        super().__init__()
        self.config = config
        self._profile_handles = []

    def init_weights(self):
        init_parameters(self, self.config)

    @property
    def device(self):
        return next(self.parameters()).device

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    # -- NVTX / torch.profiler ranges around every submodule's forward and backward --
    def save_to_state_dict(self, destination, prefix, keep_vars):
        return super()._save_to_state_dict(destination, prefix, keep_vars)

    def register_profile_hooks(self, use_nvtx: bool = True, use_record_function: bool = True,
                               profile_torch=None, profile_nsys=None):
        """``profile_torch`` / ``profile_nsys`` are the reference's names for ``use_record_function`` /
        ``use_nvtx`` (ironcore/layers/module.py:208-232)."""
        if profile_torch is not None:
            use_record_function = bool(profile_torch)
        if profile_nsys is not None:
            use_nvtx = bool(profile_nsys)
        if self._profile_handles:
            return
        nvtx_ok = use_nvtx and torch.cuda.is_available()

        def attach(mod: nn.Module, label: str):
            state = {}

            def pre_fwd(_m, _inp):
                if nvtx_ok:
                    torch.cuda.nvtx.range_push(f"Forward {label}")
                if use_record_function:
                    rf = torch.autograd.profiler.record_function(f"Forward {label}")
                    rf.__enter__()
                    state["rf"] = rf

            def post_fwd(_m, _inp, _out):
                rf = state.pop("rf", None)
                if rf is not None:
                    rf.__exit__(None, None, None)
                if nvtx_ok:
                    torch.cuda.nvtx.range_pop()

            def pre_bwd(_m, _g):
                if nvtx_ok:
                    torch.cuda.nvtx.range_push(f"Backward {label}")

            def post_bwd(_m, _gi, _go):
                if nvtx_ok:
                    torch.cuda.nvtx.range_pop()

            self._profile_handles.append(mod.register_forward_pre_hook(pre_fwd))
            self._profile_handles.append(mod.register_forward_hook(post_fwd))
            self._profile_handles.append(mod.register_full_backward_pre_hook(pre_bwd))
            self._profile_handles.append(mod.register_full_backward_hook(post_bwd))

        for name, mod in self.named_modules():
            if mod is self:
                continue
            attach(mod, f"{type(mod).__name__}({name})")

    def remove_profile_hooks(self):
        for h in self._profile_handles:
            h.remove()
        self._profile_handles = []
