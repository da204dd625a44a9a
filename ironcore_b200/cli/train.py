"""``ironcore train --config X [--<field> value ...]``.
(Behavioural reference: ironcore/cli/train.py:12-83; unlike the reference, option overrides
such as ``--tensor-model-parallel-size 2`` are accepted after ``--config``.)"""

from __future__ import annotations

import traceback
from pathlib import Path


def run_train(args, extra_argv=None) -> int:
    from ..config import apply_cli_overrides, apply_env_ranks, apply_yaml, build_arg_parser, default_config, \
        validate_config
    from ..trainer import Trainer
    from ..training_utils import forward_step, get_loss_func

    config_path = Path(args.config)
    if not config_path.exists():
        print(f"Error: Configuration file not found: {config_path}")
        return 1
    print(f"Loading training configuration from: {config_path}")
    config = default_config()
    apply_yaml(config, config_path)
    if extra_argv:
        ns = build_arg_parser().parse_args(list(extra_argv))
        apply_cli_overrides(config, ns)
    apply_env_ranks(config)
    validate_config(config)
    task_type = getattr(config.data, "task_type", "pretrain")
    loss_fn = get_loss_func(task_type)
    print(f"Task type: {task_type}, using loss function: {loss_fn.__name__}")
    if str(task_type).lower() == "grpo" or getattr(args, "rl", False):
        from ..rl.trainer import GRPOTrainer

        with GRPOTrainer(config) as trainer:
            trainer.train()
        return 0
    if str(task_type).lower() == "dpo":
        from ..rl.dpo import DPOTrainer

        trainer = DPOTrainer(config, loss_fn=loss_fn)
    else:
        trainer = Trainer(config, forward_step_func=forward_step, loss_fn=loss_fn)
    try:
        trainer.train()
        print("\nTraining completed successfully!")
        return 0
    except KeyboardInterrupt:
        print("\nTraining interrupted by user")
        return 1
    except Exception as exc:  # report and signal failure to the launcher
        print(f"\nError during training: {exc}")
        traceback.print_exc()
        return 1
    finally:
        trainer.finalize()
