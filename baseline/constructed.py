"""Constructed baselines: plain PyTorch + cuBLAS + SDPA + NCCL implementations of the workloads the
reference does not have (mixture-of-experts with expert parallelism, FSDP + Muon, GRPO rollout).
None of the framework's kernels, layers or engines is used here: ``nn.Linear`` / ``torch.matmul``
(cuBLAS), ``F.scaled_dot_product_attention``, ``dist.all_to_all_single``, ``torch.distributed.fsdp``,
``torch.optim.AdamW``. They define "what a competent PyTorch user would write" on the same model
shapes, batch and optimizer settings, and print the same JSON line as ``bench_configs.py``.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m baseline.constructed \
        --workload moe|fsdp_muon|grpo --gpus N [--steps K --warmup W --layers L]
"""

from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


# --------------------------------------------------------------------------- model
class RMSNorm(nn.Module):
    def __init__(self, d, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope_tables(seq, hd, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=device).float() / hd))
    ang = torch.outer(torch.arange(seq, device=device).float(), inv)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x, cos, sin, pos=None):
    # x: [b, h, s, hd], rotate-half convention
    if pos is not None:
        cos, sin = cos[pos], sin[pos]
    else:
        cos, sin = cos[: x.shape[2]], sin[: x.shape[2]]
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    c, s = cos.to(x.dtype), sin.to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class Attention(nn.Module):
    def __init__(self, d, heads, kv_heads, hd, qkv_bias):
        super().__init__()
        self.h, self.g, self.hd = heads, kv_heads, hd
        self.q = nn.Linear(d, heads * hd, bias=qkv_bias)
        self.kv = nn.Linear(d, 2 * kv_heads * hd, bias=qkv_bias)
        self.o = nn.Linear(heads * hd, d, bias=False)

    def forward(self, x, cos, sin, cache=None, pos=None):
        b, s, _ = x.shape
        q = self.q(x).view(b, s, self.h, self.hd).transpose(1, 2)
        k, v = self.kv(x).view(b, s, 2, self.g, self.hd).unbind(2)
        k, v = k.transpose(1, 2), v.transpose(1, 2)
        q, k = apply_rope(q, cos, sin, pos), apply_rope(k, cos, sin, pos)
        if cache is not None:
            # block KV cache kept as one contiguous tensor per layer: [b, g, max_len, hd]
            ck, cv, cur = cache
            ck[:, :, cur:cur + s] = k
            cv[:, :, cur:cur + s] = v
            k, v = ck[:, :, : cur + s], cv[:, :, : cur + s]
        rep = self.h // self.g
        if rep > 1:
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=(cache is None or s > 1))
        return self.o(y.transpose(1, 2).reshape(b, s, self.h * self.hd))


class SwiGLU(nn.Module):
    def __init__(self, d, f):
        super().__init__()
        self.up = nn.Linear(d, 2 * f, bias=False)
        self.down = nn.Linear(f, d, bias=False)

    def forward(self, x):
        g, u = self.up(x).chunk(2, -1)
        return self.down(F.silu(g) * u)


class MoE(nn.Module):
    """Top-k softmax router, E / ep local SwiGLU experts, dispatch / combine with all_to_all_single."""

    def __init__(self, d, f, experts, top_k, shared, ep_group):
        super().__init__()
        self.E, self.k, self.group = experts, top_k, ep_group
        self.ep = dist.get_world_size(ep_group) if ep_group is not None else 1
        self.e_local = experts // self.ep
        self.router = nn.Linear(d, experts, bias=False)
        self.w_up = nn.Parameter(torch.empty(self.e_local, d, 2 * f))
        self.w_down = nn.Parameter(torch.empty(self.e_local, f, d))
        self.shared = SwiGLU(d, f * shared) if shared else None
        self.aux = None

    def experts(self, x, eid):
        out = torch.empty_like(x)
        order = torch.argsort(eid, stable=True)
        counts = torch.bincount(eid, minlength=self.e_local).tolist()
        xs, off = x[order], 0
        ys = torch.empty_like(xs)
        for e, c in enumerate(counts):
            if c:
                g, u = (xs[off:off + c] @ self.w_up[e]).chunk(2, -1)
                ys[off:off + c] = (F.silu(g) * u) @ self.w_down[e]
            off += c
        out[order] = ys
        return out

    def forward(self, x):
        b, s, d = x.shape
        x2 = x.reshape(-1, d)
        probs = torch.softmax(self.router(x2).float(), -1)
        w, idx = torch.topk(probs, self.k, -1)
        f = torch.bincount(idx.reshape(-1), minlength=self.E).float() / idx.numel()
        self.aux = 0.01 * self.E * (f * probs.mean(0)).sum()
        slots = idx.reshape(-1)
        xs = x2.repeat_interleave(self.k, 0)
        if self.ep == 1:
            ys = self.experts(xs, slots)
        else:
            dest = slots // self.e_local
            order = torch.argsort(dest, stable=True)
            send = torch.bincount(dest, minlength=self.ep)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)
            in_s, out_s = send.tolist(), recv.tolist()
            er = torch.empty(sum(out_s), dtype=slots.dtype, device=x.device)
            dist.all_to_all_single(er, (slots[order] % self.e_local).contiguous(), out_s, in_s, group=self.group)
            xr = _AllToAll.apply(xs[order].contiguous(), out_s, in_s, self.group)
            yr = self.experts(xr, er)
            ys_sorted = _AllToAll.apply(yr, in_s, out_s, self.group)
            ys = torch.empty_like(ys_sorted)
            ys[order] = ys_sorted
        out = (ys.view(-1, self.k, d) * w.to(ys.dtype).unsqueeze(-1)).sum(1)
        if self.shared is not None:
            out = out + self.shared(x2)
        return out.view(b, s, d)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.splits, ctx.group = (out_splits, in_splits), group
        y = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(y, x.contiguous(), out_splits, in_splits, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        out_splits, in_splits = ctx.splits
        dx = torch.empty((sum(in_splits),) + tuple(dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        dist.all_to_all_single(dx, dy.contiguous(), in_splits, out_splits, group=ctx.group)
        return dx, None, None, None


class Block(nn.Module):
    def __init__(self, c, ep_group):
        super().__init__()
        self.n1 = RMSNorm(c["d"], c["eps"])
        self.attn = Attention(c["d"], c["heads"], c["kv_heads"], c["hd"], c.get("qkv_bias", False))
        self.n2 = RMSNorm(c["d"], c["eps"])
        if c.get("experts"):
            self.mlp = MoE(c["d"], c["ffn"], c["experts"], c["top_k"], c.get("shared", 0), ep_group)
        else:
            self.mlp = SwiGLU(c["d"], c["ffn"])

    def forward(self, x, cos, sin, cache=None, pos=None):
        x = x + self.attn(self.n1(x), cos, sin, cache, pos)
        return x + self.mlp(self.n2(x))


class Decoder(nn.Module):
    def __init__(self, c, ep_group=None):
        super().__init__()
        self.c = c
        self.emb = nn.Embedding(c["vocab"], c["d"])
        self.layers = nn.ModuleList([Block(c, ep_group) for _ in range(c["layers"])])
        self.norm = RMSNorm(c["d"], c["eps"])
        self.head = nn.Linear(c["d"], c["vocab"], bias=False)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02)

    def hidden(self, ids, caches=None, pos=None):
        cos, sin = rope_tables(self.c["max_pos"], self.c["hd"], self.c["theta"], ids.device)
        x = self.emb(ids)
        for i, layer in enumerate(self.layers):
            x = layer(x, cos, sin, None if caches is None else caches[i], pos)
        return self.norm(x)

    def forward(self, ids, labels):
        logits = self.head(self.hidden(ids)).float()
        loss = F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))
        aux = sum(l.mlp.aux for l in self.layers if isinstance(l.mlp, MoE) and l.mlp.aux is not None)
        return loss + aux if not isinstance(aux, int) else loss


SHAPES = {
    "moe": dict(layers=16, d=2048, heads=16, kv_heads=4, hd=128, ffn=1408, experts=64, top_k=6, shared=2, eps=1e-5,
                theta=1e6, vocab=32000, seq=4096, micro_batch=2, global_batch=128, max_pos=4096),
    "fsdp_muon": dict(layers=40, d=5120, heads=40, kv_heads=40, hd=128, ffn=13824, eps=1e-5, theta=1e4, vocab=32000,
                      seq=4096, micro_batch=1, global_batch=64, max_pos=4096),
    "grpo": dict(layers=28, d=1536, heads=12, kv_heads=2, hd=128, ffn=8960, eps=1e-6, theta=1e6, vocab=151936,
                 qkv_bias=True, max_pos=1024, prompts=64, prompt_len=256, group=8, new_tokens=512),
}


# --------------------------------------------------------------------------- Muon in plain PyTorch
def newton_schulz(g, steps=5):
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.bfloat16()
    t = x.shape[0] > x.shape[1]
    if t:
        x = x.t()
    x = x / (x.norm() + 1e-7)
    for _ in range(steps):
        A = x @ x.t()
        x = a * x + (b * A + c * A @ A) @ x
    return x.t() if t else x


class PlainMuonAdamW:
    """Muon on 2-D hidden matrices (full gradient gathered from the FSDP shards, orthogonalised on every rank),
    AdamW on the rest."""

    def __init__(self, model, lr=0.02, momentum=0.95, adam_lr=3e-4, wd=0.1):
        self.muon, adam = [], []
        for n, p in model.named_parameters():
            (self.muon if (p.dim() == 2 and "emb" not in n and "head" not in n) else adam).append(p)
        self.adam = torch.optim.AdamW(adam, lr=adam_lr, betas=(0.9, 0.95), weight_decay=wd)
        self.lr, self.mu = lr, momentum
        self.buf = {}

    def step(self):
        for p in self.muon:
            if p.grad is None:
                continue
            g = p.grad
            full = g.full_tensor() if hasattr(g, "full_tensor") else g
            m = self.buf.get(p)
            if m is None:
                m = self.buf[p] = torch.zeros_like(full)
            m.mul_(self.mu).add_(full)
            u = newton_schulz(full + self.mu * m)
            scale = math.sqrt(max(1.0, full.shape[0] / full.shape[1]))
            upd = (u * (self.lr * scale)).to(full.dtype)
            if hasattr(p, "to_local"):
                local = p.to_local()
                rows = local.shape[0]
                r = dist.get_rank()
                chunk = (full.shape[0] + dist.get_world_size() - 1) // dist.get_world_size()
                local.sub_(upd[r * chunk: r * chunk + rows])
            else:
                p.data.sub_(upd)
        self.adam.step()

    def zero_grad(self):
        for p in self.muon:
            p.grad = None
        self.adam.zero_grad(set_to_none=True)


# --------------------------------------------------------------------------- workloads
def run_train(args, shape, world, rank, dev):
    ep_group = None
    if args.workload == "moe" and world > 1:
        ep_group = dist.group.WORLD
    c = dict(shape)
    if args.layers:
        c["layers"] = args.layers
    torch.manual_seed(1234)
    model = Decoder(c, ep_group).to(dev).bfloat16()
    if args.workload == "fsdp_muon" and world > 1:
        from torch.distributed.fsdp import fully_shard

        for layer in model.layers:
            fully_shard(layer)
        fully_shard(model)
        opt = PlainMuonAdamW(model)
    elif args.workload == "fsdp_muon":
        opt = PlainMuonAdamW(model)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    gb = args.global_batch or c["global_batch"]
    accum = max(1, gb // (c["micro_batch"] * world))
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    batches = [torch.randint(0, c["vocab"], (c["micro_batch"], c["seq"] + 1), generator=g).to(dev) for _ in range(accum)]
    dense = [p for n, p in model.named_parameters() if "w_up" not in n and "w_down" not in n]

    def step():
        for tok in batches:
            loss = model(tok[:, :-1], tok[:, 1:])
            (loss / accum).backward()
        if args.workload == "moe" and world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in dense if p.grad is not None])
            dist.all_reduce(flat)
            flat.div_(world)
            off = 0
            for p in dense:
                if p.grad is not None:
                    n = p.grad.numel()
                    p.grad.copy_(flat[off:off + n].view_as(p.grad))
                    off += n
        if args.workload != "fsdp_muon":
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        return loss

    tokens = accum * c["micro_batch"] * world * c["seq"]
    return step, tokens, c


@torch.no_grad()
def run_grpo(args, shape, world, rank, dev):
    """Rollout only (the metric is generated tokens per second): data parallel over all ranks, contiguous KV cache,
    multinomial sampling at temperature 1."""
    c = dict(shape)
    if args.layers:
        c["layers"] = args.layers
    torch.manual_seed(1234)
    model = Decoder(c).to(dev).bfloat16().eval()
    prompts = args.prompts or max(world, c["prompts"] * world // 8)
    per_rank = max(1, prompts // world) * c["group"]
    new = args.new_tokens or c["new_tokens"]
    total = c["prompt_len"] + new
    g = torch.Generator(device="cpu").manual_seed(7 + rank)
    prompt = torch.randint(0, c["vocab"], (per_rank // c["group"], c["prompt_len"]), generator=g).to(dev)
    prompt = prompt.repeat_interleave(c["group"], 0)

    @torch.no_grad()      # (a decorator on run_grpo alone would not cover this closure, which runs later)
    def step():
        caches = [(torch.empty(per_rank, c["kv_heads"], total, c["hd"], dtype=torch.bfloat16, device=dev),
                   torch.empty(per_rank, c["kv_heads"], total, c["hd"], dtype=torch.bfloat16, device=dev), 0)
                  for _ in range(c["layers"])]
        h = model.hidden(prompt, caches)
        cur = c["prompt_len"]
        logits = model.head(h[:, -1]).float()
        out = []
        for t in range(new):
            tok = torch.multinomial(torch.softmax(logits, -1), 1)
            out.append(tok)
            if t == new - 1:
                break
            caches = [(ck, cv, cur) for ck, cv, _ in caches]
            pos = torch.full((1,), cur, device=dev, dtype=torch.long)
            h = model.hidden(tok, caches, pos)
            cur += 1
            logits = model.head(h[:, -1]).float()
        return torch.cat(out, 1)

    return step, per_rank * world * new, c


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True, choices=sorted(SHAPES))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--global-batch", dest="global_batch", type=int, default=0)
    ap.add_argument("--prompts", type=int, default=0)
    ap.add_argument("--new-tokens", dest="new_tokens", type=int, default=0)
    ap.add_argument("--tiny", action="store_true", help="shrink every dimension (functional check on CPU)")
    args = ap.parse_args(argv)
    if args.tiny:
        for sh in SHAPES.values():
            sh.update(layers=2, d=64, heads=4, kv_heads=2, hd=16, ffn=32, vocab=256, max_pos=64)
            if "seq" in sh:
                sh.update(seq=32, global_batch=4, micro_batch=1)
            if "experts" in sh:
                sh.update(experts=4, top_k=2, shared=1)
            if "prompts" in sh:
                sh.update(prompts=8, prompt_len=8, group=2, new_tokens=4)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo")
    fn = run_grpo if args.workload == "grpo" else run_train
    step, tokens, c = fn(args, SHAPES[args.workload], world, rank, dev)

    def sync():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync()
    t0 = time.perf_counter()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for _ in range(args.steps):
        step()
    if cuda:
        e1.record()
    sync()
    ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    if rank == 0:
        print(json.dumps({
            "impl": "constructed (plain PyTorch + cuBLAS + SDPA + NCCL)", "workload": args.workload,
            "metric": "grpo_rollout_tokens_per_s" if args.workload == "grpo" else "train_tokens_per_s",
            "value": tokens / (ms_per_step / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "config": {k: v for k, v in c.items() if not isinstance(v, (list, dict))},
            "memory_gib": torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else None}), flush=True)
    import faulthandler

    # a stalled teardown is reported (stacks on stderr, exit status 1), never passed off as success
    faulthandler.dump_traceback_later(45.0, exit=True)
    if world > 1:
        dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()
    faulthandler.dump_traceback_later(45.0, exit=True)


if __name__ == "__main__":
    main()
