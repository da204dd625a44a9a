"""Where a step of the flash attention backward kernel goes, per role, in cycles.

Builds ``csrc/flash_bwd.cu`` (+ ``csrc/flash_fwd.cu`` for the shared tensor-map helpers) once more with
``-DICB_FB_TRACE`` into ``benchmarks/_build/libicb_fbtrace.so``: the kernel then adds ``clock64`` differences
around every wait of its TMA thread, its MMA thread and one softmax thread to 16 device counters. The product
library is not touched and contains none of this. Needs ``nvcc`` and one B200.

    python -m benchmarks.flash_bwd_trace [--cases b,s,hq,hkv,hd ...]

Prints one JSON line per case: kernel time (CUDA events), steps (one step = one 128 x 128 block pair),
average cycles per step of every counter, and the largest difference to the product kernel's gradients.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import shutil
import subprocess
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
BUILD = Path(__file__).resolve().parent / "_build"
LIB = BUILD / "libicb_fbtrace.so"
NAMES = ["tma_wait_q_empty", "tma_wait_do_empty", "mma_wait_q_full", "mma_wait_do_full", "mma_wait_dq_empty",
         "mma_wait_p_full", "softmax_wait_s_full", "softmax_s_full_to_ds_published", "softmax_wait_dq_full",
         "softmax_dq_drain", "cta_total", "softmax_wait_staging_tile", "tma_wait_stage_free", "softmax_wait_dp_full"]


def build() -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    BUILD.mkdir(exist_ok=True)
    srcs = [ROOT / "csrc" / "flash_bwd.cu", ROOT / "csrc" / "flash_fwd.cu"]
    if LIB.exists() and all(LIB.stat().st_mtime > s.stat().st_mtime for s in srcs):
        return LIB
    cmd = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
           "-std=c++17", "-DICB_FB_TRACE", "-diag-suppress", "177", "-I", str(ROOT / "csrc"), *map(str, srcs), "-o", str(LIB)]
    subprocess.run(cmd, check=True)
    return LIB


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", nargs="*", default=["1,4096,32,32,128", "1,4096,4,4,128", "2,4096,16,4,128"],
                    help="batch,seq,heads,kv_heads,head_dim")
    args = ap.parse_args(argv)
    from ironcore_b200.ops import attention, native
    from ironcore_b200.ops.native import dtype_code, ptr, stream_ptr

    lib = C.CDLL(str(build()))
    P, I, L, F = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    lib.icb_flash_bwd.argtypes = [P] * 11 + [I, I, L, I, I, I, L, L, L, L, P, I, F, I, P, P, F, P]
    lib.icb_flash_bwd.restype = I
    lib.icb_flash_bwd_trace_read.argtypes = [P, I]
    for case in args.cases:
        b, s, hq, hkv, hd = (int(v) for v in case.split(","))
        t = b * s
        torch.manual_seed(0)
        qkv = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda").bfloat16()
        dout = torch.randn(t, hq * hd, device="cuda").bfloat16()
        out, lse = attention.flash_fwd(qkv, hq, hkv, hd, s)
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(hq, t, device="cuda")
        dq_acc = torch.empty(t, hq * hd, device="cuda")
        es, base, dbase, st = 2, qkv.data_ptr(), dqkv.data_ptr(), qkv.stride(0)

        def run():
            rc = lib.icb_flash_bwd(ptr(dout), base, base + hq * hd * es, base + (hq + hkv) * hd * es, ptr(out), ptr(lse),
                                   dbase, dbase + hq * hd * es, dbase + (hq + hkv) * hd * es, ptr(delta), ptr(dq_acc),
                                   b, s, t, hq, hkv, hd, st, st, st, st, None, 1, hd ** -0.5, dtype_code(qkv.dtype),
                                   ptr(native.status_tensor(qkv.device)), stream_ptr(), 0.0, None)
            if rc:
                raise RuntimeError(f"icb_flash_bwd (traced build) returned {rc}")

        for _ in range(3):
            run()
        torch.cuda.synchronize()
        buf = (C.c_ulonglong * 16)()
        lib.icb_flash_bwd_trace_read(buf, 1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        native.check_status()
        lib.icb_flash_bwd_trace_read(buf, 1)
        v = list(buf)
        steps = max(v[15], 1)
        ref = attention.flash_bwd(dout, qkv, out, lse, hq, hkv, hd, s)
        print(json.dumps({"case": {"batch": b, "seq": s, "heads": hq, "kv_heads": hkv, "head_dim": hd},
                          "traced_kernel_ms": e0.elapsed_time(e1), "steps": v[15], "ctas": v[14],
                          "cycles_per_step": {n: round(x / steps) for n, x in zip(NAMES, v)},
                          "max_abs_diff_vs_product_kernel": (ref.float() - dqkv.float()).abs().max().item()}),
              flush=True)


if __name__ == "__main__":
    main()
