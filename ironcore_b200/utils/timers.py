"""Named timers (host wall clock and device CUDA events), memory report, profiler ranges.
(Behavioural reference: ironcore/utils.py:146-265.)"""

from __future__ import annotations

import contextlib
import functools
import time
from typing import Dict, List, Optional

import torch


class _HostTimer:
    def __init__(self, name):
        self.name, self.laps, self._t0 = name, [], None

    def start(self, sync: bool = False):
        if sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self._t0 = time.perf_counter()

    def stop(self, sync: bool = False):
        if self._t0 is None:
            return 0.0
        if sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - self._t0
        self.laps.append(dt)
        self._t0 = None
        return dt

    def elapsed(self, reset: bool = False) -> float:
        """Mean lap time in seconds."""
        m = sum(self.laps) / len(self.laps) if self.laps else 0.0
        if reset:
            self.laps = []
        return m

    def last(self) -> float:
        return self.laps[-1] if self.laps else 0.0

    def reset(self):
        self.laps, self._t0 = [], None


class Timer:
    """``timer.start("iter") ... timer.stop("iter"); timer.elapsed("iter")`` -> mean of laps."""

    def __init__(self):
        self.timers: Dict[str, _HostTimer] = {}

    def __call__(self, name) -> _HostTimer:
        if name not in self.timers:
            self.timers[name] = _HostTimer(name)
        return self.timers[name]

    def start(self, name, sync=False):
        self(name).start(sync)

    def stop(self, name, sync=False):
        return self(name).stop(sync)

    def elapsed(self, name, reset=False):
        return self(name).elapsed(reset)

    def last(self, name):
        return self(name).last()

    def reset(self, name=None):
        for n in ([name] if name else list(self.timers)):
            self(n).reset()

    # -- the reference's remaining timer calls (ironcore/utils.py:153-216) --
    def register(self, name):
        if name in self.timers:
            raise KeyError(f"Requested timer ({name}) is already registered")
        self.timers[name] = _HostTimer(name)

    def get(self, name) -> float:
        """Mean lap time of ``name`` in seconds; a running timer is stopped first."""
        if name not in self.timers:
            raise KeyError(f"Not initialized timer ({name}) is requested")
        t = self.timers[name]
        if t._t0 is not None:
            t.stop()
        return t.elapsed()

    def get_summary(self) -> Dict[str, float]:
        return {n: t.elapsed() for n, t in self.timers.items() if t.laps}

    def reset_all(self):
        self.reset()

    def stop_all(self):
        for t in self.timers.values():
            if t._t0 is not None:
                t.stop()


class DeviceTimer:
    """CUDA-event timer on the current stream; ``elapsed_ms`` synchronises on the end event."""

    def __init__(self):
        self._pairs: List = []
        self._start = None

    def start(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._start.record()

    def stop(self):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self._pairs.append((self._start, end))
        self._start = None

    def elapsed_ms(self, reset: bool = True) -> List[float]:
        out = []
        for s, e in self._pairs:
            e.synchronize()
            out.append(s.elapsed_time(e))
        if reset:
            self._pairs = []
        return out


def get_memory_usage(device=None) -> Dict[str, float]:
    """Allocated / reserved / peak memory in MiB."""
    if not torch.cuda.is_available():
        return {"allocated": 0.0, "reserved": 0.0, "max_allocated": 0.0, "max_reserved": 0.0}
    mib = 1024.0 * 1024.0
    return {
        "allocated": torch.cuda.memory_allocated(device) / mib,
        "reserved": torch.cuda.memory_reserved(device) / mib,
        "max_allocated": torch.cuda.max_memory_allocated(device) / mib,
        "max_reserved": torch.cuda.max_memory_reserved(device) / mib,
    }


@contextlib.contextmanager
def profile_context(name: str, nvtx: bool = True):
    """NVTX range + torch.profiler record_function around a block."""
    use_nvtx = nvtx and torch.cuda.is_available()
    if use_nvtx:
        torch.cuda.nvtx.range_push(name)
    with torch.autograd.profiler.record_function(name):
        try:
            yield
        finally:
            if use_nvtx:
                torch.cuda.nvtx.range_pop()


def profile_function(name: Optional[str] = None):
    def deco(fn):
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def wrapped(*a, **k):
            with profile_context(label):
                return fn(*a, **k)

        return wrapped

    return deco
