"""Reference arm of the benchmark: the unmodified IronCore reference (installed into
``baseline/_ref``) driven through its own public API — ``MainConfig`` -> ``Trainer`` ->
``Trainer.train_step`` — on the same model / batch / optimizer settings as ``bench.py``.

The reference cannot run offline as shipped, so five import-time shims are applied without
touching its source:
  1. ``ironcore.global_vars.build_tokenizer`` -> a vocab-size-only tokenizer object (the real
     one downloads from the HuggingFace hub);
  2. ``ironcore.trainer.get_data_iterator`` -> a synthetic uniform-token iterator built in
     pinned host memory (the real one needs preprocessed dataset files);
  3. ``torch.nn.RMSNorm`` accepts and ignores the ``bias=`` keyword the reference passes
     (without it ``ln_type: rmsnorm`` raises ``TypeError`` in the reference);
  4. a stub ``mlflow`` module if mlflow is not installed (imported at module load);
  5. ``BaseModule.device`` falls back to the current CUDA device for modules without
     parameters: the reference's flash-attention path asks its parameter-free ``Attention``
     module for ``self.device`` and raises ``StopIteration`` as shipped. With this shim the
     reference runs its faster flash path; if that path still fails, the arm falls back to the
     reference's standard attention with its own per-layer activation recompute (otherwise the
     materialised [1,32,4096,4096] scores of 32 layers do not fit), and reports which mode ran.
What is timed is the reference's stock path: its model, its flash-attn call, its autocast
context, its TP layers with NCCL all-reduce (no sequence parallelism and a replicated AdamW,
because the reference has neither SP nor ZeRO-1).
"""

from __future__ import annotations

import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


class _StubTokenizer:
    def __init__(self, vocab_size: int, unit: int, tp: int):
        self.vocab_size = vocab_size
        mult = unit * tp
        self.padded_vocab_size = (vocab_size + mult - 1) // mult * mult
        self.eos_token_id = vocab_size - 1
        self.eod_token_id = vocab_size - 1
        self.pad_token_id = vocab_size - 1
        self.eos_token = "<eos>"


def _install_shims(vocab_size: int):
    import torch

    if "mlflow" not in sys.modules:
        try:
            import mlflow  # noqa: F401
        except Exception:
            sys.modules["mlflow"] = types.ModuleType("mlflow")
    base_rms = torch.nn.RMSNorm
    if not getattr(base_rms, "_accepts_bias_kw", False):
        class RMSNormCompat(base_rms):
            _accepts_bias_kw = True

            def __init__(self, *a, bias=None, **k):
                super().__init__(*a, **k)

        torch.nn.RMSNorm = RMSNormCompat
    sys.path.insert(0, REF_DIR)
    import ironcore.global_vars as gv
    import ironcore.trainer as tr

    def build_tokenizer(config):
        return _StubTokenizer(vocab_size, config.trainer.vocab_padding_unit, config.trainer.tensor_model_parallel_size)

    gv.build_tokenizer = build_tokenizer
    import ironcore.layers.module as ref_module

    def _device(self):
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")

    ref_module.BaseModule.device = property(_device)
    return gv, tr


def run_reference(args, model_kw, global_batch, seq_len, metric) -> int:
    if not os.path.isdir(os.path.join(REF_DIR, "ironcore")):
        return _unavailable("baseline/_ref is missing: install the reference with pip --target baseline/_ref")
    import torch

    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        return _unavailable(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    try:
        gv, tr = _install_shims(model_kw["vocab_size"])
        from ironcore.config import MainConfig, _config_validation
        from ironcore.config import (DataConfig, InitConfig, ModelConfig, OperationConfig, OptimConfig,
                                     ParallelConfig, TrainerConfig, UtilsConfig)
        from ironcore.training_utils import forward_step, loss_func
    except Exception as exc:  # pragma: no cover
        return _unavailable(f"reference import failed: {type(exc).__name__}: {exc}")

    rank = int(os.environ["RANK"])
    cfg = MainConfig(model=ModelConfig(), init=InitConfig(), optim=OptimConfig(), data=DataConfig(),
                     parallel=ParallelConfig(), trainer=TrainerConfig(), operation=OperationConfig(),
                     utils=UtilsConfig())
    m = cfg.model
    m.d_model, m.d_ffn, m.num_layers = model_kw["d_model"], model_kw["d_ffn"], model_kw["num_layers"]
    m.num_attention_heads = model_kw["num_attention_heads"]
    m.num_attention_groups = model_kw["num_attention_groups"]
    m.head_dim = model_kw["head_dim"]
    m.max_seq_len = seq_len
    m.max_position_embeddings = seq_len
    m.dropout_embd = m.dropout_attn = m.dropout_mlp = 0.0
    m.precision = "bfloat16"
    m.reset_position_ids = False
    m.reset_attention_mask = False
    m.positional_embedding.type = "rope"
    m.positional_embedding.base = 10000
    m.untie_embed = True
    m.no_bias = True
    m.ln_type = "rmsnorm"
    m.ln_eps = 1e-5
    m.activation_type = "swiglu"
    m.name = "llama"
    cfg.data.vocab_size = model_kw["vocab_size"]
    cfg.trainer.micro_batch_size = 1
    cfg.trainer.train_batch_size = global_batch
    cfg.trainer.gradient_accumulation_steps = None
    cfg.trainer.tensor_model_parallel_size = world
    cfg.trainer.use_flash_attn = True
    cfg.trainer.model_path = ""
    cfg.trainer.log_interval = 10 ** 9
    cfg.operation.train_steps = 10 ** 6
    cfg.operation.no_save = True
    cfg.optim.max_lr, cfg.optim.min_lr = 3e-4, 3e-5
    cfg.optim.adam_beta1, cfg.optim.adam_beta2 = 0.9, 0.95
    cfg.optim.weight_decay, cfg.optim.clip_grad = 0.1, 1.0
    cfg.init.init_std, cfg.init.seed = 0.02, 1234
    cfg.parallel.rank, cfg.parallel.world_size = rank, world
    cfg.parallel.local_rank = int(os.environ["LOCAL_RANK"])
    cfg.utils.report_memory_usage = False
    _config_validation(cfg)
    accum = cfg.trainer.gradient_accumulation_steps

    dev = torch.device("cuda", cfg.parallel.local_rank)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device="cpu").manual_seed(1234)
    pool = [torch.empty((1, seq_len + 1), dtype=torch.int64).pin_memory() for _ in range(2 * accum)]
    state = {"i": 0, "resident": None}

    def host_batches():
        while True:
            buf = pool[state["i"] % len(pool)]
            state["i"] += 1
            torch.randint(0, model_kw["vocab_size"], buf.shape, generator=gen, out=buf)
            yield {"input_ids": buf[:, :-1], "labels": buf[:, 1:]}

    def resident_batches():
        items = []
        g2 = torch.Generator(device="cpu").manual_seed(1234)
        for _ in range(accum):
            tok = torch.randint(0, model_kw["vocab_size"], (1, seq_len + 1), generator=g2).to(dev)
            items.append({"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()})
        k = 0
        while True:
            yield items[k % accum]
            k += 1

    iters = {"train": resident_batches(), "eval": None, "test": None}
    tr.get_data_iterator = lambda config: iters

    def attempt(flash: bool):
        """Build the reference trainer and run one probing step in the given attention mode."""
        gv.GLOBAL_STATES = None
        cfg.trainer.use_flash_attn = flash
        cfg.operation.activation_recompute = not flash
        t = tr.Trainer(cfg, forward_step, loss_func)
        t.train_step(0)
        torch.cuda.synchronize()
        return t

    mode = "flash_attn (reference flash path with the parameter-free-module device shim)"
    trainer = None
    try:
        trainer = attempt(True)
    except Exception as exc:
        first_error = f"{type(exc).__name__}: {str(exc)[:160]}"
        import gc

        trainer = None
        gc.collect()
        torch.cuda.empty_cache()
        try:
            trainer = attempt(False)
            mode = f"standard attention + activation recompute (flash path failed: {first_error})"
        except Exception as exc2:
            import traceback

            traceback.print_exc()
            return _unavailable(f"reference train_step failed in both attention modes: {first_error} / "
                                f"{type(exc2).__name__}: {str(exc2)[:160]}")
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(HERE))
    from bench import ClockSampler

    def barrier_sync():
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tokens_per_step = global_batch * seq_len
    try:
        for s in range(args.warmup):
            trainer.train_step(s)
        barrier_sync()
        sampler = ClockSampler(torch.cuda.current_device())
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier_sync()
        e0.record()
        for s in range(args.steps):
            trainer.train_step(args.warmup + s)
        e1.record()
        barrier_sync()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist.get_world_size() > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t.item()) / args.steps
        # end to end: pinned host batches, loss read back every step
        trainer.data_iterator["train"] = host_batches()
        loss, _, _ = trainer.train_step(0)
        float(loss)
        barrier_sync()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        last = None
        for s in range(args.steps):
            loss, _, _ = trainer.train_step(s)
            last = float(loss)
        f1.record()
        barrier_sync()
        t2 = torch.tensor([f0.elapsed_time(f1)], device=dev)
        if dist.get_world_size() > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e = tokens_per_step / (float(t2.item()) / args.steps / 1e3)
        clocks = sampler.stop() if rank == 0 else None
    except torch.cuda.OutOfMemoryError as exc:
        return _unavailable(f"reference ran out of device memory on this config: {str(exc)[:120]}")
    if rank == 0:
        out = {
            "impl": "reference", "metric": metric, "value": tokens_per_step / (ms_per_step / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": "llama-7b-shape (32L, d4096, 32h x 128, ffn 11008 swiglu, vocab 32000)",
                       "global_batch": global_batch, "seq_len": seq_len, "micro_batch": 1,
                       "parallelism": f"tp{world} (reference TP: no sequence parallelism, replicated AdamW)",
                       "attention_mode": mode,
                       "shims": "offline tokenizer stub, synthetic data iterator, RMSNorm bias kwarg, "
                                "device property of parameter-free modules"},
            "clocks": clocks,
            "ms_per_step_x_sm_mhz": (ms_per_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": accum * 2 * seq_len * 8,
                    "d2h_bytes_per_step": 4, "last_loss": last},
            "gpu_launches": 0,
            "memory_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }
        print(json.dumps(out), flush=True)
    from bench import guarded_teardown

    guarded_teardown(trainer._finialize_process)
    return 0
