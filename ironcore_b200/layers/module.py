"""Base module: dtype/device properties and recursive profiler ranges.
(Behavioural reference: ironcore/layers/module.py:19-232.)"""

from __future__ import annotations

import torch
import torch.nn as nn


class BaseModule(nn.Module):
    def __init__(self, config=None):
        super().__init__()
        self.config = config
        self._profile_handles = []

    @property
    def device(self):
        return next(self.parameters()).device

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    # -- NVTX / torch.profiler ranges around every submodule's forward and backward --
    def register_profile_hooks(self, use_nvtx: bool = True, use_record_function: bool = True):
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
