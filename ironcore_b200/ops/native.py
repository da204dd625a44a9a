"""ctypes loader for the in-tree sm_100a kernel library.

The library exports a plain C ABI (``icb_*``): raw device pointers, sizes, and the
CUDA stream as an opaque pointer. This module declares the signatures, loads the
``.so`` once, and raises loudly if a CUDA device is present but the library is
missing or a kernel reports an error — there is no silent eager fallback on GPU.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_LAUNCHES = 0  # number of native kernel entry points invoked (one or more device launches each)

P = C.c_void_p
I = C.c_int
L = C.c_longlong
F = C.c_float

_SIGNATURES = {
    "icb_gemm": [P, P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, I, I, P, L, P, I, P],
    "icb_norm_bwd_parts": [I],
    "icb_norm_fwd": [P, P, P, P, P, P, P, P, I, I, F, F, I, I, P, P],
    "icb_norm_bwd": [P, P, P, P, P, P, P, P, P, P, I, I, F, I, I, I, I, P, P],
    "icb_rope": [P, P, P, I, I, I, L, L, I, F, F, I, I, I, I, P, I],
    "icb_glu_fwd": [P, P, L, I, I, I, I, P, P],
    "icb_glu_bwd": [P, P, P, L, I, I, I, I, P, P],
    "icb_act_fwd": [P, P, L, I, I, P],
    "icb_act_bwd": [P, P, P, L, I, I, P],
    "icb_embedding_fwd": [P, P, P, P, P, I, I, I, I, I, I, P],
    "icb_embedding_bwd": [P, P, P, I, I, I, I, I, P],
    "icb_ce_stats": [P, P, P, P, P, I, I, L, I, I, I, P],
    "icb_ce_grad": [P, P, P, P, I, I, L, I, I, I, P],
    "icb_adam": [P, P, P, P, L, F, F, F, F, F, F, F, P, I, I, P],
    "icb_sumsq_parts": [L],
    "icb_sumsq": [P, L, P, P, I, I, P],
    "icb_clip_coef": [P, F, P, P, P],
}


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "_native" / "libironcore_b200.so"


def available() -> bool:
    """True when the native library can be used (CUDA device present and .so loadable)."""
    if not torch.cuda.is_available():
        return False
    return load(strict=True) is not None


def load(strict: bool = False):
    """Load (building if necessary) the native library. Returns None on CPU-only hosts
    unless ``strict``."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not path.exists() or os.environ.get("ICB_REBUILD") == "1":
            from . import build as _build

            _build.build()
        try:
            lib = C.CDLL(str(path))
        except OSError as exc:  # pragma: no cover - depends on host
            if strict or torch.cuda.is_available():
                raise RuntimeError(f"cannot load native kernel library {path}: {exc}") from exc
            return None
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue
            fn.argtypes = argtypes
            fn.restype = I
        _LIB = lib
        return _LIB


def register(name: str, argtypes) -> None:
    """Declare one more exported symbol (used by modules that own extra kernels)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name, None)   # an optional entry point may be absent from an older build
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = I


def launches() -> int:
    return _LAUNCHES


def add_launches(n: int) -> None:
    """Account for kernels launched by replaying a captured CUDA graph."""
    global _LAUNCHES
    _LAUNCHES += int(n)


def reset_launches() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def call(name: str, *args) -> int:
    """Invoke an exported function; raise on a non-zero return code."""
    global _LAUNCHES
    lib = load(strict=True)
    fn = getattr(lib, name)
    rc = fn(*args)
    _LAUNCHES += 1
    if rc != 0:
        raise RuntimeError(f"native kernel {name} failed with code {rc}")
    return rc


def query(name: str, *args) -> int:
    """Invoke an exported function that returns a value rather than a status."""
    lib = load(strict=True)
    return getattr(lib, name)(*args)


def ptr(t):
    """Device pointer of a tensor (or NULL for None)."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError as exc:
        raise TypeError(f"unsupported dtype for native kernels: {dt}") from exc


# ---------------------------------------------------------------------------
# Device status word: kernels that give up on a bounded wait write a code here.
# ---------------------------------------------------------------------------
_STATUS = {}

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free smem stage",
    3: "timeout waiting for an accumulator",
    4: "timeout waiting for the epilogue",
    5: "timeout waiting for a peer flag",
    6: "timeout waiting for a local flag",
    7: "bad argument",
}


def status_tensor(device=None) -> torch.Tensor:
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = dev.index
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _STATUS[key] = t
    return t


def set_wait_limit_us(microseconds: int, device=None) -> None:
    """How long one device-side wait (mbarrier phase, peer flag, tile counter) may last before the
    kernel gives up, writes a status code and returns. 0 restores the default of two seconds."""
    status_tensor(device)[1] = int(microseconds)


def clear_status(device=None) -> None:
    """Reset the status code and detail; the configured wait limit stays."""
    t = status_tensor(device)
    t[0] = 0
    t[2] = 0


def check_status(device=None) -> None:
    """Synchronising check of the device status word; raises if any kernel reported an error."""
    t = status_tensor(device)
    code, _limit, detail, _ = (int(v) for v in t.tolist())
    if code != 0:
        clear_status(device)
        raise RuntimeError(f"native kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')} "
                           f"(detail {detail})")
