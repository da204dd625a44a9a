"""Evaluate a checkpoint on the tasks named under ``data.eval_datasets`` (HellaSwag-style multiple choice).

    HELLASWAG_PATH=./data/hellaswag_val.jsonl python examples/evaluation.py --config configs/example.yaml \
        --tasks hellaswag --samples 200
"""

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--tasks", default="hellaswag", help="comma-separated task names")
    ap.add_argument("--samples", type=int, default=None)
    ap.add_argument("--batch-size", dest="batch_size", type=int, default=1)
    args = ap.parse_args()

    from ironcore_b200 import global_vars as G
    from ironcore_b200.checkpoint import load_checkpoint
    from ironcore_b200.config import apply_env_ranks, apply_yaml, default_config, validate_config
    from ironcore_b200.eval.evaluator import get_evaluators
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    config = default_config()
    apply_yaml(config, Path(args.config))
    apply_env_ranks(config)
    validate_config(config)
    G.set_global_states(config)
    mesh.initialize_process(config)
    mesh.initialize_model_parallel(config.trainer.tensor_model_parallel_size)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    model = LanguageModel(config, device=dev).eval()
    step = load_checkpoint(config, model)
    tasks = get_evaluators([{"name": t.strip()} for t in args.tasks.split(",") if t.strip()],
                           batch_size=args.batch_size, num_samples=args.samples)
    for task in tasks:
        result = task.process(model)
        if mesh.is_rank_zero():
            print(f"[step {step}] {task.name}: " + ", ".join(f"{k} = {v:.3f}" for k, v in result.items()))
    mesh.finalize_process()


if __name__ == "__main__":
    main()
