"""Flash attention micro-benchmark against the FlashAttention-2 package (when importable)."""

from __future__ import annotations

import json

import torch


def bench_attention(results, quick: bool = False):
    from ironcore_b200.ops import attention
    from .kernels import _flush_buffer, time_cuda

    flush = _flush_buffer()
    cases = [("llama7b", 1, 4096, 32, 32, 128), ("llama7b_tp8", 1, 4096, 4, 4, 128), ("gqa", 2, 4096, 16, 4, 128),
             ("gpt2", 4, 1024, 12, 12, 64), ("long", 1, 16384, 8, 8, 128)]
    if quick:
        cases = cases[:1]
    try:
        from flash_attn import flash_attn_func
    except Exception:
        flash_attn_func = None
    for name, b, s, hq, hkv, hd in cases:
        t = b * s
        qkv = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda").bfloat16()
        dout = torch.randn(t, hq * hd, device="cuda").bfloat16()
        out, lse = attention.flash_fwd(qkv, hq, hkv, hd, s)
        fwd_flops = 4.0 * b * s * s * hq * hd / 2
        ms_f = time_cuda(lambda: attention.flash_fwd(qkv, hq, hkv, hd, s), flush=flush)
        ms_b = time_cuda(lambda: attention.flash_bwd(dout, qkv, out, lse, hq, hkv, hd, s), flush=flush)
        rec = {"kernel": "flash_attn", "case": name, "b": b, "s": s, "hq": hq, "hkv": hkv, "hd": hd,
               "fwd_ms": ms_f, "fwd_tflops": fwd_flops / ms_f / 1e9, "bwd_ms": ms_b,
               "bwd_tflops": 2.5 * fwd_flops / ms_b / 1e9}
        if flash_attn_func is not None:
            x = qkv.view(b, s, hq + 2 * hkv, hd)
            q = x[:, :, :hq].contiguous().requires_grad_(True)
            k = x[:, :, hq:hq + hkv].contiguous().requires_grad_(True)
            v = x[:, :, hq + hkv:].contiguous().requires_grad_(True)
            ref_f = time_cuda(lambda: flash_attn_func(q, k, v, causal=True), flush=flush)
            o = flash_attn_func(q, k, v, causal=True)
            do = dout.view(b, s, hq, hd)
            ref_b = time_cuda(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True), flush=flush)
            rec.update({"fa2_fwd_ms": ref_f, "fa2_fwd_tflops": fwd_flops / ref_f / 1e9, "fa2_bwd_ms": ref_b,
                        "fa2_bwd_tflops": 2.5 * fwd_flops / ref_b / 1e9})
        results.append(rec)
        print(json.dumps(rec), flush=True)
