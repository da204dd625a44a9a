"""``ironcore export --config X --output DIR [--step N] [--pytorch] [--shard-bytes B]``: write the checkpoint under
``trainer.model_path`` (the latest one, or step N) as a HuggingFace directory (weights + ``config.json``).
Run it with the parallel layout the checkpoint needs (one process for a merged checkpoint; under ``torchrun`` with
the training layout for per-rank checkpoints): tensor- and expert-parallel shards are gathered, rank 0 writes.
(Behavioural reference: ``export_to_huggingface`` of ironcore/checkpointing/hf_interop.py:304-558, which the
reference offers as a function only.)"""

from __future__ import annotations

from pathlib import Path


def run_export(args, extra_argv=None) -> int:
    import torch
    import torch.distributed as dist

    from ..checkpoint import load_checkpoint
    from ..checkpoint.hf_interop import export_to_huggingface
    from ..config import apply_cli_overrides, apply_env_ranks, apply_yaml, build_arg_parser, default_config, \
        validate_config
    from ..global_vars import set_global_states
    from ..models.language_model import LanguageModel
    from ..parallel import mesh

    path = Path(args.config)
    if not path.exists():
        print(f"Error: Configuration file not found: {path}")
        return 1
    config = default_config()
    apply_yaml(config, path)
    if extra_argv:
        apply_cli_overrides(config, build_arg_parser().parse_args(list(extra_argv)))
    apply_env_ranks(config)
    validate_config(config)
    set_global_states(config)
    mesh.initialize_process(config)
    mesh.initialize_model_parallel(config.trainer.tensor_model_parallel_size,
                                   expert_model_parallel_size=config.parallel.expert_model_parallel_size,
                                   timeout_in_minutes=float(config.parallel.timeout_minute or 10.0))
    try:
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        model = LanguageModel(config, device=dev)
        step = load_checkpoint(config, model, step=args.step)
        if step is None or step < 0:
            print(f"Error: no checkpoint under {config.trainer.model_path!r}")
            return 1
        out = export_to_huggingface(model, config, args.output, safe_serialization=not args.pytorch,
                                    max_shard_bytes=args.shard_bytes or None)
        if mesh.is_rank_zero():
            print(f"exported step {step} -> {out}")
        return 0
    finally:
        if dist.is_initialized():
            mesh.finalize_process()
