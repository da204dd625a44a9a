"""Micro-benchmarks of the native kernels against their library counterparts.

``python -m benchmarks.kernels [--out FILE] [--quick]`` times each kernel
with CUDA events (3 warm-up launches, L2 flushed between timed launches by writing a
256 MiB buffer) and prints one JSON line per case with achieved TFLOP/s or GB/s.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def _flush_buffer():
    return torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush=None) -> float:
    """Median milliseconds of fn() over ``iters`` launches."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(results, quick: bool, two_sm: bool = False):
    from ironcore_b200.ops import kernels

    shapes = [
        ("qkv_7b", 4096, 12288, 4096), ("out_7b", 4096, 4096, 4096), ("gateup_7b", 4096, 22016, 4096),
        ("down_7b", 4096, 4096, 11008), ("head_7b", 4096, 32000, 4096), ("square_8k", 8192, 8192, 8192),
        ("qkv_tp8", 4096, 1536, 4096), ("down_tp8", 4096, 4096, 1376),
    ]
    if quick:
        shapes = shapes[:2]
    flush = _flush_buffer()
    two_sm_ok = two_sm and kernels.two_sm_available()
    for name, m, n, k in shapes:
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = torch.randn(k, n, device="cuda").bfloat16()
        dy = torch.randn(m, n, device="cuda").bfloat16()
        flops = 2.0 * m * n * k
        for label, fn, ref in (
            ("fwd", lambda **kw: kernels.mm_nn(x, w, **kw), lambda: torch.matmul(x, w)),
            ("dgrad", lambda **kw: kernels.mm_nt(dy, w, **kw), lambda: torch.matmul(dy, w.t())),
            ("wgrad", lambda **kw: kernels.mm_tn(x, dy, **kw), lambda: torch.matmul(x.t(), dy)),
        ):
            ours = time_cuda(fn, flush=flush)
            lib = time_cuda(ref, flush=flush)
            pair = time_cuda(lambda: fn(two_sm=True), flush=flush) if two_sm_ok else None
            results.append({"kernel": "gemm", "case": f"{name}_{label}", "m": m, "n": n, "k": k, "ms": ours,
                            "tflops": flops / ours / 1e9, "cublas_ms": lib, "cublas_tflops": flops / lib / 1e9,
                            "two_sm_ms": pair, "two_sm_tflops": (flops / pair / 1e9) if pair else None})
            print(json.dumps(results[-1]), flush=True)


def bench_elementwise(results, quick: bool):
    from ironcore_b200.ops import kernels

    flush = _flush_buffer()
    d = 4096
    w = torch.ones(d, device="cuda").bfloat16()
    # two row counts: at 16384 rows (0.13 GB per tensor) a launch takes 50-80 us and the few microseconds of launch
    # and event overhead are a tenth of it; 65536 rows show the kernel's own rate
    for m in (16384, 65536):
        x = torch.randn(m, d, device="cuda").bfloat16()
        ms = time_cuda(lambda: kernels.norm_fwd(x, w, None, 1e-5, True), flush=flush)
        results.append({"kernel": "rmsnorm_fwd", "rows": m, "d": d, "ms": ms, "gbs": 2 * x.numel() * 2 / ms / 1e6})
        print(json.dumps(results[-1]), flush=True)
        y, h, mean, rstd = kernels.norm_fwd(x, w, None, 1e-5, True)
        ms = time_cuda(lambda: kernels.norm_bwd(x, x, w, mean, rstd, True, False), flush=flush)
        results.append({"kernel": "rmsnorm_bwd", "rows": m, "d": d, "ms": ms, "gbs": 3 * x.numel() * 2 / ms / 1e6})
        print(json.dumps(results[-1]), flush=True)
        del x, y, h
    m = 16384
    g = torch.randn(m, 2 * 11008, device="cuda").bfloat16()
    ms = time_cuda(lambda: kernels.glu_fwd(g, "swiglu"), flush=flush)
    results.append({"kernel": "swiglu_fwd", "ms": ms, "gbs": 1.5 * g.numel() * 2 / ms / 1e6})
    print(json.dumps(results[-1]), flush=True)
    n = 512 * 1024 * 1024
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    gr = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    mm = torch.zeros(n, device="cuda")
    vv = torch.zeros(n, device="cuda")
    ms = time_cuda(lambda: kernels.adam_step_(p, gr, mm, vv, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                              weight_decay=0.1, step=1), iters=5)
    results.append({"kernel": "adam", "ms": ms, "gbs": n * 22 / ms / 1e6})
    print(json.dumps(results[-1]), flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--two-sm", dest="two_sm", action="store_true", help="also time the CTA-pair (cta_group::2) GEMM")
    ap.add_argument("--only", default=None, help="comma separated subset: gemm,elementwise,attention")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("no CUDA device", file=sys.stderr)
        return 1
    results = []
    only = set(args.only.split(",")) if args.only else None
    if only is None or "gemm" in only:
        bench_gemm(results, args.quick, args.two_sm)
    if only is None or "elementwise" in only:
        bench_elementwise(results, args.quick)
    if only is None or "attention" in only:
        try:
            from .attention import bench_attention
        except ImportError:
            bench_attention = None
        if bench_attention is not None:
            bench_attention(results, args.quick)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
