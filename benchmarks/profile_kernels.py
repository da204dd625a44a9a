"""Launch one native kernel a few times on a small (but larger-than-L2) case, for ``ncu``.

    python -m benchmarks.profile_kernels --kernel gemm|gemm_wgrad|flash_fwd|flash_bwd|rmsnorm|swiglu|adam|ag_gemm|gemm_rs|zero_step|moe_dispatch

``ag_gemm`` / ``gemm_rs`` / ``zero_step`` / ``moe_dispatch`` run the fused compute+collective kernels on a one-rank group (the peer table
points at this GPU's own buffers), which exercises the same code path — copy warps, flags, P2P
epilogue, in-kernel reduction — inside a single process that a profiler can wrap."""

from __future__ import annotations

import argparse
import os

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args(argv)
    from ironcore_b200.ops import attention, kernels, native

    dev = "cuda"
    torch.manual_seed(0)
    k = args.kernel
    if k in ("gemm", "gemm_wgrad"):
        m, n, kk = 8192, 4096, 4096
        x = torch.randn(m, kk, device=dev).bfloat16()
        w = torch.randn(kk, n, device=dev).bfloat16()
        dy = torch.randn(m, n, device=dev).bfloat16()
        fn = (lambda: kernels.mm_nn(x, w)) if k == "gemm" else (lambda: kernels.mm_tn(x, dy))
    elif k in ("flash_fwd", "flash_bwd"):
        b, s, h, hd = 1, 4096, 32, 128
        qkv = torch.randn(b * s, 3 * h * hd, device=dev).bfloat16()
        out, lse = attention.flash_fwd(qkv, h, h, hd, s)
        dout = torch.randn_like(out)
        fn = (lambda: attention.flash_fwd(qkv, h, h, hd, s)) if k == "flash_fwd" else \
            (lambda: attention.flash_bwd(dout, qkv, out, lse, h, h, hd, s))
    elif k == "rmsnorm":
        x = torch.randn(32768, 4096, device=dev).bfloat16()
        w = torch.ones(4096, device=dev).bfloat16()
        fn = lambda: kernels.norm_fwd(x, w, None, 1e-5, True)
    elif k == "swiglu":
        x = torch.randn(16384, 2 * 11008, device=dev).bfloat16()
        fn = lambda: kernels.glu_fwd(x, "swiglu")
    elif k == "adam":
        n = 256 * 1024 * 1024
        p = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        g = torch.zeros(n, device=dev)
        mm, vv = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        fn = lambda: kernels.adam_step_(p, g, mm, vv, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1)
    elif k in ("ag_gemm", "gemm_rs"):
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        from ironcore_b200.parallel.fused_comm import FusedTP

        t, d = 8192, 4096
        ws = FusedTP(t, d, dist.group.WORLD)
        if k == "ag_gemm":
            x = torch.randn(t, d, device=dev).bfloat16()
            w = torch.randn(d, 4096, device=dev).bfloat16()
            fn = lambda: ws.ag_gemm(x, w, a_major=0, b_major=1, n=4096)
        else:
            a = torch.randn(t, 2048, device=dev).bfloat16()
            w = torch.randn(2048, d, device=dev).bfloat16()
            res = torch.randn(t, d, device=dev).bfloat16()
            fn = lambda: ws.gemm_rs(a, w, b_major=1, residual=res)
    elif k in ("zero_step", "moe_dispatch"):
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29578")
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        if k == "zero_step":
            from ironcore_b200.optim.fused_zero import FusedZeroStep

            n = 128 * 1024 * 1024      # 256 MiB of bf16 parameters, 512 MiB of fp32 gradients

            class _Group:
                total = n

            fz = FusedZeroStep(dist.group.WORLD)
            pbuf, gbuf = fz.allocate(_Group, torch.bfloat16, torch.float32)
            gbuf.normal_()
            m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            regions = [(0, n, 1.0, 0.1, 1.0)]
            fn = lambda: fz.step(regions, 0, m, v, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, step_size=1e-3,
                                 grad_scale=1.0, clip=1.0)
        else:
            from ironcore_b200.parallel.fused_moe import FusedEP

            t, d, e, kk = 8192, 2048, 64, 6
            ws = FusedEP(dist.group.WORLD, e, kk, t, d, torch.bfloat16, 1.0)
            x = torch.randn(t, d, device=dev).bfloat16()
            expert = torch.randint(0, e, (t * kk,), device=dev, dtype=torch.int32)
            w = torch.rand(t, kk, device=dev)

            def fn():
                xp, dest, seg, tile_expert, counts = ws.dispatch(x, expert)
                ws.pull(xp, expert, dest, t, weight=w.reshape(-1).contiguous())
    else:
        raise SystemExit(f"unknown kernel {k}")
    for _ in range(args.iters):
        fn()
    torch.cuda.synchronize()
    native.check_status()
    print(f"profile_kernels {k}: ok")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
