"""Command-line entry: ``ironcore {train,preprocess,inspect,rollout,export} ...`` (also ``python -m ironcore_b200``).
(Behavioural reference: ironcore/__main__.py:16-89.)"""

from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="ironcore", description="ironcore_b200: B200-native LLM training framework")
    sub = parser.add_subparsers(dest="command")

    p_pre = sub.add_parser("preprocess", help="tokenize datasets into data.bin / data.idx.npy")
    p_pre.add_argument("--config", required=True, help="dataset YAML (UniversalDataConfig)")
    p_pre.add_argument("--inspect", action="store_true", help="inspect the outputs after preprocessing")
    p_pre.add_argument("--only-inspect", action="store_true", help="inspect existing outputs, do not preprocess")
    p_pre.add_argument("--preview", type=int, default=0, help="number of samples to preview")

    p_ins = sub.add_parser("inspect", help="integrity checks, statistics and previews of preprocessed data")
    p_ins.add_argument("--config", required=True, help="dataset YAML (UniversalDataConfig)")
    p_ins.add_argument("--preview", type=int, default=0, help="number of samples to preview")

    p_train = sub.add_parser("train", help="run training from a YAML configuration")
    p_train.add_argument("--config", required=True, help="training YAML")
    p_train.add_argument("--rl", action="store_true", help="run the GRPO loop instead of pre-training")

    p_roll = sub.add_parser("rollout", help="sample from a model on the paged KV cache")
    p_roll.add_argument("--config", required=True)
    p_roll.add_argument("--prompt", default=None)
    p_roll.add_argument("--max-new-tokens", type=int, default=64)

    p_exp = sub.add_parser("export", help="write a native checkpoint as a HuggingFace directory")
    p_exp.add_argument("--config", required=True, help="training YAML of the run that wrote the checkpoint")
    p_exp.add_argument("--output", required=True, help="directory to write")
    p_exp.add_argument("--step", type=int, default=None, help="checkpoint step (default: the latest)")
    p_exp.add_argument("--pytorch", action="store_true", help="pytorch_model.bin instead of safetensors")
    p_exp.add_argument("--shard-bytes", dest="shard_bytes", type=int, default=0, help="maximum bytes per weight file")

    args, extra = parser.parse_known_args(argv)
    if args.command == "preprocess":
        from .cli.preprocess import run_preprocess

        return run_preprocess(args) or 0
    if args.command == "inspect":
        from .cli.preprocess import run_preprocess

        args.only_inspect, args.inspect = True, True       # same code path as `preprocess --only-inspect`
        return run_preprocess(args) or 0
    if args.command == "train":
        from .cli.train import run_train

        return run_train(args, extra)
    if args.command == "rollout":
        from .cli.rollout import run_rollout

        return run_rollout(args, extra)
    if args.command == "export":
        from .cli.export import run_export

        return run_export(args, extra)
    parser.print_help()
    return 1


if __name__ == "__main__":
    sys.exit(main())
