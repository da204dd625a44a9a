"""Sample text from a checkpoint (or a freshly initialised model) on the paged KV cache.

    python examples/generate_text.py --config configs/example.yaml --prompt "The weather today" \
        --max-new-tokens 64 --temperature 0.8 --top-k 50 --top-p 0.95

On a GPU the decode loop runs as a captured CUDA graph per step over the block KV cache with the paged
decode-attention kernel; on CPU the same engine runs on the PyTorch oracle ops.
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
    ap.add_argument("--prompt", default="")
    ap.add_argument("--max-new-tokens", dest="max_new_tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", dest="top_k", type=int, default=0)
    ap.add_argument("--top-p", dest="top_p", type=float, default=1.0)
    ap.add_argument("--num-samples", dest="num_samples", type=int, default=1)
    args = ap.parse_args()

    from ironcore_b200 import global_vars as G
    from ironcore_b200.checkpoint import load_checkpoint
    from ironcore_b200.config import apply_env_ranks, apply_yaml, default_config, validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh
    from ironcore_b200.rl import RolloutEngine

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
    tok = G.get_tokenizer()
    ids = tok.encode(args.prompt) if args.prompt else [tok.eos_token_id]
    prompts = torch.tensor([ids] * args.num_samples, dtype=torch.long)
    engine = RolloutEngine(model, config, max_seqs=args.num_samples, max_seq_len=len(ids) + args.max_new_tokens)
    out, _ = engine.generate(prompts, args.max_new_tokens, args.temperature, args.top_k, args.top_p)
    if mesh.is_rank_zero():
        print(f"[checkpoint step {step}]")
        for i in range(args.num_samples):
            print(f"--- sample {i} ---")
            print(args.prompt + tok.decode(out[i, len(ids):].tolist()))
    mesh.finalize_process()


if __name__ == "__main__":
    main()
