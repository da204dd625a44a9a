"""Shared helpers for the test suite: tiny configs and multi-process launch on CPU ranks."""

from __future__ import annotations

import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp


def tiny_config(family="gpt2", **model_overrides):
    from ironcore_b200.config import default_config

    c = default_config()
    base = dict(name=family, d_model=64, d_ffn=128, num_layers=2, num_attention_heads=4, max_seq_len=32,
                max_position_embeddings=32, precision="fp32", vocab_size=512, dropout_embd=0.0, dropout_attn=0.0,
                dropout_mlp=0.0)
    if family.startswith("llama") or family.startswith("qwen"):
        base.update(ln_type="rmsnorm", activation_type="swiglu", no_bias=True, untie_embed=True,
                    num_attention_groups=2, positional_embedding={"type": "rope"})
    base.update(model_overrides)
    c.model(**base)
    c.data(task_type="synthetic", vocab_size=512)
    c.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None, log_interval=1,
              vocab_padding_unit=8)
    c.operation(train_steps=3)
    c.init(init_std=0.02, seed=7)
    c.optim(max_lr=1e-3, warmup_steps=0, clip_grad=1.0)
    c.parallel.world_size = 1
    c.parallel.rank = 0
    return c


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, errq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        import torch.distributed as dist

        dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_distributed(fn, world: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` on ``world`` CPU processes over Gloo; re-raise failures."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    for p in procs:
        if p.is_alive():
            p.terminate()
            failed.append("timeout")
        elif p.exitcode != 0:
            failed.append(f"exit {p.exitcode}")
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    if failed or msgs:
        raise AssertionError("distributed run failed: " + "; ".join(failed) + "\n" +
                             "\n".join(f"[rank {r}]\n{tb}" for r, tb in msgs))


# ------------------------------------------------------------------ GPU ranks as child processes
def _gpu_worker(rank, world, port, module_name, fn_name, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        import importlib

        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        fn = getattr(importlib.import_module(module_name), fn_name)
        fn(rank, world)
        torch.cuda.synchronize()
        from ironcore_b200.ops import native

        native.check_status()
        dist.barrier()
        dist.destroy_process_group()
        out_q.put((rank, "ok"))
    except Exception:
        out_q.put((rank, traceback.format_exc()))


def spawn_gpu_ranks(module_name: str, fn_name: str, world: int = 2, timeout: float = 150.0):
    """Run ``module.fn(rank, world)`` as ``world`` child processes, one CUDA device and one NCCL rank each
    (``world = 1`` gives a one-rank group whose peer tables point at the GPU's own buffers)."""
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, world, port, module_name, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    results = []
    while not q.empty():
        results.append(q.get())
    bad = [r for r in results if r[1] != "ok"]
    for p in procs:
        if p.is_alive():
            p.terminate()
            bad.append((-1, "timeout"))
    assert not bad and len(results) == world, "\n".join(f"[rank {r}] {m}" for r, m in bad)
