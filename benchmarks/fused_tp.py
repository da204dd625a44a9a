"""Micro-benchmark of the fused TP kernels against the NCCL + GEMM composition.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m benchmarks.fused_tp [--tokens 4096 --width 4096 --ffn 11008]

Times (CUDA events, max over ranks, L2 flushed between launches) the four call sites of a
Llama-shape layer at tensor-parallel size N and prints one JSON line per case with the
achieved time, the NCCL-composition time and the roofline (slower of GEMM time at the
measured bf16 peak and bytes over NVLink at the measured peer bandwidth).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--trace", action="store_true", help="per-CTA timestamps of the fused all-gather kernel")
    ap.add_argument("--cases", default="", help="comma-separated case names to run (default: all)")
    ap.add_argument("--helpers", action="store_true",
                    help="the epilogue warps of every CTA push chunks of the gather shard too (default: two copy warps)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironcore_b200.ops import kernels, native
    from ironcore_b200.parallel.fused_comm import FusedTP

    t, d, f = args.tokens, args.width, args.ffn
    ws = FusedTP(t, d, dist.group.WORLD, num_slots=1)    # NVLS form when the fabric offers multicast
    ws_p2p = FusedTP(t, d, dist.group.WORLD, nvls=False, num_slots=1) if ws.nvls else ws   # plain P2P stores / loads
    if args.helpers:
        ws.push_helpers = ws_p2p.push_helpers = True
    rows = t // world
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    peak_tflops, link_gbs = 1414.0, 770.0

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        times = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        times.sort()
        v = torch.tensor([times[len(times) // 2]], device="cuda")
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    cases = []
    # column-parallel forward: AG(x)[t, d] @ W[d, n_local]
    for name, n_local in (("qkv_fwd", 3 * d // world), ("gate_up_fwd", 2 * f // world)):
        n_local = (n_local + 7) // 8 * 8
        x = torch.randn(rows, d, device="cuda").bfloat16()
        w = torch.randn(d, n_local, device="cuda").bfloat16()
        full = torch.empty(t, d, device="cuda", dtype=torch.bfloat16)

        def fused(ws=ws, x=x, w=w, n_local=n_local):
            return ws.ag_gemm(x, w, a_major=0, b_major=1, n=n_local)

        def nccl(x=x, w=w, full=full):
            dist.all_gather_into_tensor(full, x)
            return kernels.mm_nn(full, w)

        def gemm_only(w=w, full=full):
            kernels.mm_nn(full, w)

        flops = 2.0 * t * d * n_local
        wire = (world - 1) * rows * d * 2
        cases.append((name, "ag_gemm", fused, nccl, gemm_only, flops, wire))
    # column-parallel weight gradient: AG(x)^T @ dy[t, n_local] (reduction over the gathered tokens)
    for name, n_local in (("qkv_wgrad", 3 * d // world), ("gate_up_wgrad", 2 * f // world)):
        n_local = (n_local + 7) // 8 * 8
        x = torch.randn(rows, d, device="cuda").bfloat16()
        dy = torch.randn(t, n_local, device="cuda").bfloat16()
        full = torch.empty(t, d, device="cuda", dtype=torch.bfloat16)

        def fused(ws=ws, x=x, dy=dy, n_local=n_local):
            return ws.ag_gemm(x, dy, a_major=1, b_major=1, n=n_local)

        def nccl(x=x, dy=dy, full=full):
            dist.all_gather_into_tensor(full, x)
            return kernels.mm_tn(full, dy)

        def gemm_only(dy=dy, full=full):
            kernels.mm_tn(full, dy)

        cases.append((name, "ag_gemm_wgrad", fused, nccl, gemm_only, 2.0 * t * d * n_local, (world - 1) * rows * d * 2))
    # row-parallel forward: (x[t, k_local] @ W[k_local, d]) -> RS
    for name, k_local in (("attn_out_fwd", d // world), ("down_fwd", f // world)):
        k_local = (k_local + 7) // 8 * 8
        a = torch.randn(t, k_local, device="cuda").bfloat16()
        w = torch.randn(k_local, d, device="cuda").bfloat16()
        out = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)

        def fused(ws=ws, a=a, w=w):
            return ws.gemm_rs(a, w, b_major=1)

        def nccl(a=a, w=w, out=out):
            y = kernels.mm_nn(a, w)
            dist.reduce_scatter_tensor(out, y)
            return out

        def gemm_only(a=a, w=w):
            kernels.mm_nn(a, w)

        flops = 2.0 * t * d * k_local
        wire = (world - 1) * rows * d * 2
        cases.append((name, "gemm_rs", fused, nccl, gemm_only, flops, wire))
    # chains across a norm boundary: row-parallel GEMM -> reduce-scatter (+residual) -> RMSNorm -> all-gather ->
    # column-parallel GEMM. "fused": one producer kernel (GEMM + reduce + norm + push) and one consumer kernel that
    # only waits; "separate": the two fused GEMM+collective kernels with a norm kernel between them.
    for name, k_local, n_local in (("attn_out_norm_gate_up", d // world, 2 * f // world),
                                   ("down_norm_qkv", f // world, 3 * d // world)):
        k_local, n_local = (k_local + 7) // 8 * 8, (n_local + 7) // 8 * 8
        a = torch.randn(t, k_local, device="cuda").bfloat16()
        w = (torch.randn(k_local, d, device="cuda") / (k_local * world) ** 0.5).bfloat16()
        res = torch.randn(rows, d, device="cuda").bfloat16()
        gamma = torch.ones(d, device="cuda").bfloat16()
        w2 = torch.randn(d, n_local, device="cuda").bfloat16()
        out = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)
        full = torch.empty(t, d, device="cuda", dtype=torch.bfloat16)

        def fused(ws=ws, a=a, w=w, res=res, gamma=gamma, w2=w2, n_local=n_local):
            slot = ws.slots[0]
            ws.gemm_rs(a, w, b_major=1, residual=res, norm=(gamma, 1e-5, 0.0, slot))
            return ws.ag_gemm(slot.local, w2, a_major=0, b_major=1, n=n_local, slot=slot, pushed=True)

        def separate(ws=ws, a=a, w=w, res=res, gamma=gamma, w2=w2, n_local=n_local):
            h = ws.gemm_rs(a, w, b_major=1, residual=res)
            y = kernels.norm_fwd(h, gamma, None, 1e-5, True)[0]
            return ws.ag_gemm(y, w2, a_major=0, b_major=1, n=n_local)

        def nccl(a=a, w=w, res=res, gamma=gamma, w2=w2, out=out, full=full):
            y = kernels.mm_nn(a, w)
            dist.reduce_scatter_tensor(out, y)
            yn = kernels.norm_fwd(out, gamma, None, 1e-5, True, residual=res)[0]
            dist.all_gather_into_tensor(full, yn)
            return kernels.mm_nn(full, w2)

        def gemm_only(a=a, w=w, gamma=gamma, w2=w2, full=full, out=out):
            kernels.mm_nn(a, w)
            kernels.norm_fwd(out, gamma, None, 1e-5, True)
            kernels.mm_nn(full, w2)

        flops = 2.0 * t * d * (k_local + n_local)
        wire = 2 * (world - 1) * rows * d * 2
        cases.append((name, "rs_norm_ag_chain", fused, nccl, gemm_only, flops, wire))
        cases.append((name + "_separate_kernels", "rs_norm_ag_chain", separate, nccl, gemm_only, flops, wire))
    # the same boundaries in backward: column-parallel dgrad -> reduce-scatter -> RMSNorm backward (+ residual
    # gradient) -> all-gather -> row-parallel dgrad
    for name, n_col, k_row in (("gate_up_dgrad_normbwd_attn_out_dgrad", 2 * f // world, d // world),
                               ("qkv_dgrad_normbwd_down_dgrad", 3 * d // world, f // world)):
        n_col, k_row = (n_col + 7) // 8 * 8, (k_row + 7) // 8 * 8
        dy = torch.randn(t, n_col, device="cuda").bfloat16()
        w_col = (torch.randn(d, n_col, device="cuda") / (n_col * world) ** 0.5).bfloat16()   # [in = d, out]
        w_row = torch.randn(k_row, d, device="cuda").bfloat16()                              # [in, out = d]
        xin = torch.randn(rows, d, device="cuda").bfloat16()
        gamma = torch.ones(d, device="cuda").bfloat16()
        rstd = kernels.norm_fwd(xin, gamma, None, 1e-5, True)[3]
        dres = torch.randn(rows, d, device="cuda").bfloat16()
        out = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)
        full = torch.empty(t, d, device="cuda", dtype=torch.bfloat16)

        def fused(ws=ws, dy=dy, w_col=w_col, w_row=w_row, xin=xin, gamma=gamma, rstd=rstd, dres=dres, k_row=k_row):
            dx, _dn = ws.gemm_rs_norm_bwd(dy, w_col, b_major=0, residual=dres, gamma=gamma, w_offset=0.0, rstd=rstd,
                                          x=xin)
            return ws.ag_gemm(dx, w_row, a_major=0, b_major=0, n=k_row, pushed=True)

        def separate(ws=ws, dy=dy, w_col=w_col, w_row=w_row, xin=xin, gamma=gamma, rstd=rstd, dres=dres, k_row=k_row):
            dn = ws.gemm_rs(dy, w_col, b_major=0)
            dx = kernels.norm_bwd(dn, xin, gamma, None, rstd, True, False, dres_in=dres)[0]
            return ws.ag_gemm(dx, w_row, a_major=0, b_major=0, n=k_row)

        def nccl(dy=dy, w_col=w_col, w_row=w_row, xin=xin, gamma=gamma, rstd=rstd, dres=dres, out=out, full=full):
            y = kernels.mm_nt(dy, w_col)
            dist.reduce_scatter_tensor(out, y)
            dx = kernels.norm_bwd(out, xin, gamma, None, rstd, True, False, dres_in=dres)[0]
            dist.all_gather_into_tensor(full, dx)
            return kernels.mm_nt(full, w_row)

        def gemm_only(dy=dy, w_col=w_col, w_row=w_row, xin=xin, gamma=gamma, rstd=rstd, out=out, full=full):
            kernels.mm_nt(dy, w_col)
            kernels.norm_bwd(out, xin, gamma, None, rstd, True, False)
            kernels.mm_nt(full, w_row)

        flops = 2.0 * t * d * (n_col + k_row)
        wire = 2 * (world - 1) * rows * d * 2
        cases.append((name, "rs_normbwd_ag_chain", fused, nccl, gemm_only, flops, wire))
        cases.append((name + "_separate_kernels", "rs_normbwd_ag_chain", separate, nccl, gemm_only, flops, wire))
    wanted = {c for c in args.cases.split(",") if c}
    for name, kind, fused, nccl, gemm_only, flops, wire in cases:
        if wanted and name not in wanted:
            continue
        ref = nccl().float()
        err = max(float((fused(ws=w_).float() - ref).abs().max()) for w_ in {id(ws): ws, id(ws_p2p): ws_p2p}.values())
        scale = float(ref.abs().max())
        if args.trace and kind.startswith("ag_gemm"):
            native.register("icb_set_ag_debug", [native.P])
            dbg = torch.zeros(148 * 4, dtype=torch.int64, device="cuda")
            for w_ in ({id(ws): ws, id(ws_p2p): ws_p2p}.values()):
                for _ in range(3):
                    fused(ws=w_)
                torch.cuda.synchronize()
                flush.zero_()
                dist.barrier()
                torch.cuda.synchronize()
                native.call("icb_set_ag_debug", dbg.data_ptr())
                fused(ws=w_)
                torch.cuda.synchronize()
                native.call("icb_set_ag_debug", None)
                t = dbg.view(148, 4).cpu().double()
                t0 = t[:, 0].min()
                def stat(col):
                    v = (t[:, col][t[:, col] > 0] - t0) / 1e3
                    return [round(float(v.min()), 1), round(float(v.median()), 1), round(float(v.max()), 1)] if v.numel() else None
                print(json.dumps({"trace": name, "rank": rank, "nvls_ag": w_.nvls_ag, "us_since_first_cta_start": {
                    "cta_start": stat(0), "push_done": stat(1), "first_remote_block_ready": stat(2), "epilogue_done": stat(3)}}),
                    flush=True)
                dbg.zero_()
        tf = timeit(fused)
        tp = timeit(lambda: fused(ws=ws_p2p)) if ws_p2p is not ws else tf
        tn = timeit(nccl)
        tg = timeit(gemm_only)
        roof_ms = max(flops / (peak_tflops * 1e9), wire / (link_gbs * 1e6))
        if rank == 0:
            print(json.dumps({"case": name, "kind": kind, "world": world, "nvls": ws.nvls, "fused_ms": tf,
                              "fused_p2p_ms": tp, "max_abs_err_vs_nccl": err, "ref_abs_max": scale, "nccl_plus_gemm_ms": tn,
                              "gemm_only_ms": tg, "roofline_ms": roof_ms, "fraction_of_roofline": roof_ms / tf,
                              "wire_mb": wire / 1e6, "gflop": flops / 1e9}), flush=True)
    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    import faulthandler

    faulthandler.dump_traceback_later(45.0, exit=True)   # a stuck communicator teardown ends with exit status 1
    dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()


if __name__ == "__main__":
    main()
