"""``ironcore rollout --config X [--prompt TEXT] [--max-new-tokens N]``: sample from a (checkpointed
or freshly initialised) model on the paged KV cache."""

from __future__ import annotations

from pathlib import Path

import torch


def run_rollout(args, extra_argv=None) -> int:
    from .. import global_vars as G
    from ..checkpoint import load_checkpoint
    from ..config import apply_cli_overrides, apply_env_ranks, apply_yaml, build_arg_parser, default_config, \
        validate_config
    from ..models import LanguageModel
    from ..parallel import mesh
    from ..rl import RolloutEngine

    config = default_config()
    apply_yaml(config, Path(args.config))
    if extra_argv:
        apply_cli_overrides(config, build_arg_parser().parse_args(list(extra_argv)))
    apply_env_ranks(config)
    validate_config(config)
    G.set_global_states(config)
    mesh.initialize_process(config)
    mesh.initialize_model_parallel(config.trainer.tensor_model_parallel_size)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    model = LanguageModel(config, device=dev).eval()
    load_checkpoint(config, model)
    tok = G.get_tokenizer()
    rl = config.rl
    if args.prompt:
        ids = torch.tensor([tok.encode(args.prompt)], dtype=torch.long)
    else:
        ids = torch.randint(0, model.vocab_size, (1, rl.prompt_len))
    engine = RolloutEngine(model, config, max_seqs=ids.shape[0], max_seq_len=ids.shape[1] + args.max_new_tokens)
    out, _ = engine.generate(ids, args.max_new_tokens, rl.temperature, rl.top_k, rl.top_p)
    if mesh.is_rank_zero():
        print(tok.decode(out[0, ids.shape[1]:].tolist()))
    return 0
