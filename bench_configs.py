"""Throughput of the other named workloads (the flagship Llama-7B TP benchmark is ``bench.py``).

    python bench_configs.py --workload moe|fsdp_muon|grpo|gpt2|llama7b [--gpus N --steps K --warmup W --layers L]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_configs.py --workload moe --gpus N

Each workload loads its preset from ``configs/`` and adapts only what depends on the number of GPUs
(expert-parallel size = min(8, N); FSDP over N ranks; GRPO TP2 x DP(N/2), TP1 on one GPU); the global
batch stays the preset's unless ``--global-batch`` is given. ``--layers``
runs a shallower model of the same layer shape when the full depth does not fit the GPUs given, and
is reported in the JSON line. ``llama7b --tp T`` is the headline model on a TP x DP mesh (T-way tensor +
sequence parallel inside each replica, data parallel with ZeRO-1 optimizer-state sharding across replicas:
e.g. TP2 x DP4 on 8 GPUs), next to ``bench.py``'s TP = N layout. Synthetic uniform tokens, random-init
weights, device timing with CUDA events (max over ranks), one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
PRESET = {"moe": "configs/baseline_moe_ep8.yaml", "fsdp_muon": "configs/baseline_llama13b_fsdp_muon.yaml",
          "grpo": "configs/baseline_grpo_qwen.yaml", "gpt2": "configs/example.yaml", "llama7b": None}


def build_config(args, world: int):
    from ironcore_b200.config import apply_env_ranks, apply_yaml, default_config, validate_config

    os.chdir(ROOT)
    if args.workload == "llama7b":
        from bench import build_config as headline_config

        tp = args.tp or world
        if world % tp:
            raise SystemExit(f"--tp {tp} does not divide {world} GPUs")
        c = headline_config(tp, args.steps)
        overlap = bool(args.overlap_grad_reduce) and world > tp
        # (the overlapped reduction needs the autograd hooks of an eager backward pass: no graph replay)
        c.trainer(tensor_model_parallel_size=tp, cuda_graph=tp > 1 and not overlap)
        c.parallel(world_size=world, sequence_parallel=tp > 1, zero_stage=1, overlap_grad_reduce=overlap)
        c.trainer.gradient_accumulation_steps = None
        if args.layers:
            c.model.num_layers = args.layers
        if args.global_batch:
            c.trainer.train_batch_size = args.global_batch
        apply_env_ranks(c)
        validate_config(c)
        return c
    c = default_config()
    apply_yaml(c, PRESET[args.workload])
    c.trainer(log_interval=10 ** 9, model_path="")
    c.operation(train_steps=10 ** 6, no_save=True)
    c.utils(report_memory_usage=False)
    c.data(task_type="synthetic")
    if c.data.vocab_size in (None, 51200) and c.model.vocab_size:
        c.data.vocab_size = c.model.vocab_size
    if args.layers:
        c.model.num_layers = args.layers
    if args.workload == "moe":
        c.parallel.expert_model_parallel_size = min(8, world)
    elif args.workload == "fsdp_muon":
        c.parallel.use_fsdp = world > 1
        c.parallel.fsdp_fused_gather = bool(args.fsdp_fused_gather) and world > 1
    elif args.workload == "grpo":
        tp = 2 if world >= 2 else 1
        c.trainer.tensor_model_parallel_size = tp
        dp = world // tp
        # 64 prompts on 8 GPUs; fewer GPUs roll out proportionally fewer prompts (same work per GPU)
        c.rl.num_prompts = args.prompts if args.prompts else max(dp, c.rl.num_prompts * world // 8)
        c.rl.num_prompts -= c.rl.num_prompts % dp
        if args.new_tokens:
            c.rl.max_new_tokens = args.new_tokens
    elif args.workload == "gpt2":
        c.trainer.train_batch_size = c.trainer.micro_batch_size * world * 4
        c.data.vocab_size = 50257
        c.model.vocab_size = 50257
    if args.global_batch:
        c.trainer.train_batch_size = args.global_batch
    c.trainer.gradient_accumulation_steps = None
    apply_env_ranks(c)
    validate_config(c)
    return c


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True, choices=sorted(PRESET))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = preset)")
    ap.add_argument("--global-batch", dest="global_batch", type=int, default=0,
                    help="sequences per optimizer step (0 = the preset's: strong scaling over --gpus)")
    ap.add_argument("--prompts", type=int, default=0, help="GRPO: prompts per rollout batch (0 = preset scaled by GPUs)")
    ap.add_argument("--new-tokens", dest="new_tokens", type=int, default=0, help="GRPO: generated tokens per sample")
    ap.add_argument("--tp", type=int, default=0, help="llama7b: tensor-parallel size (0 = all GPUs); the rest is DP")
    ap.add_argument("--fsdp-fused-gather", dest="fsdp_fused_gather", action="store_true",
                    help="fsdp_muon: parameter gathers as P2P / multicast kernels instead of NCCL all-gathers")
    ap.add_argument("--overlap-grad-reduce", dest="overlap_grad_reduce", action="store_true",
                    help="llama7b with --tp below the GPU count: all-reduce gradient buckets behind the last backward pass")
    args = ap.parse_args(argv)
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29617")
    sys.path.insert(0, ROOT)
    from bench import ClockSampler
    from ironcore_b200.ops import native
    from ironcore_b200.parallel import mesh

    cfg = build_config(args, world)
    if args.workload == "grpo":
        from ironcore_b200.rl.trainer import GRPOTrainer

        trainer = GRPOTrainer(cfg)
    else:
        from ironcore_b200.trainer import Trainer

        trainer = Trainer(cfg)
    dev = trainer.device

    def barrier_sync():
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for s in range(args.warmup):
        trainer.train_step(s)
    barrier_sync()
    native.reset_launches()
    sampler = ClockSampler(torch.cuda.current_device())
    if mesh.get_rank() == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier_sync()
    e0.record()
    rollout_s, last = 0.0, None
    for s in range(args.steps):
        last = trainer.train_step(args.warmup + s)
        if args.workload == "grpo":
            rollout_s += last["rollout_s"]       # device-timed, already the maximum over ranks
    e1.record()
    barrier_sync()
    t = torch.tensor([e0.elapsed_time(e1), rollout_s * 1e3], device=dev)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t[0]) / args.steps
    clocks = sampler.stop() if mesh.get_rank() == 0 else None
    native.check_status()
    if mesh.get_rank() == 0:
        m = cfg.model
        if args.workload == "grpo":
            gen = cfg.rl.num_prompts * cfg.rl.group_size * cfg.rl.max_new_tokens
            metric, value = "grpo_rollout_tokens_per_s", gen / (float(t[1]) / args.steps / 1e3)
            extra = {"step_ms_including_update": ms_per_step, "sequences": cfg.rl.num_prompts * cfg.rl.group_size,
                     "prompt_len": cfg.rl.prompt_len, "new_tokens": cfg.rl.max_new_tokens,
                     "reward_mean": last.get("reward_mean"), "kl_mean": last.get("kl_mean")}
        else:
            tokens = cfg.trainer.train_batch_size * m.max_seq_len
            metric, value = "train_tokens_per_s", tokens / (ms_per_step / 1e3)
            extra = {"last_loss": float(last[0])}
        print(json.dumps({
            "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "dtype": m.precision,
            "data": "synthetic", "impl": "ironcore_b200", "workload": args.workload,
            "config": {"preset": PRESET[args.workload] or "bench.py model", "model": m.name, "layers": m.num_layers,
                       "layers_overridden": bool(args.layers), "d_model": m.d_model,
                       "global_batch": cfg.trainer.train_batch_size, "micro_batch": cfg.trainer.micro_batch_size,
                       "seq_len": m.max_seq_len, "tp": cfg.trainer.tensor_model_parallel_size,
                       "ep": cfg.parallel.expert_model_parallel_size, "fsdp": cfg.parallel.use_fsdp,
                       "fsdp_fused_gather": bool(getattr(cfg.parallel, "fsdp_fused_gather", False)),
                       "overlap_grad_reduce": bool(getattr(cfg.parallel, "overlap_grad_reduce", False)),
                       "optimizer": cfg.optim.optimizer, "zero_stage": cfg.parallel.zero_stage},
            "clocks": clocks, "gpu_launches": native.launches(),
            "memory_gib": torch.cuda.max_memory_allocated() / 2 ** 30, **extra}), flush=True)
    from bench import guarded_teardown

    guarded_teardown(trainer.finalize)


if __name__ == "__main__":
    main()
