"""Small driver for profilers: a few layers of a named model shape, a couple of micro-batch
forward + backward passes and one optimizer step on one GPU.

    python -m benchmarks.profile_step --layers 2 --iters 2 [--shape llama7b|qwen1p5b|gpt2]

Meant to be wrapped by ``ncu --metrics gpu__time_duration.sum`` (one pass, every launch) or by
``ncu --set full -k regex:<kernel> -c 3`` for one kernel; it keeps the device footprint to a few GB."""

from __future__ import annotations

import argparse

import torch

SHAPES = {
    "llama7b": dict(d_model=4096, num_attention_heads=32, num_attention_groups=32, head_dim=128, d_ffn=11008,
                    max_seq_len=4096, vocab_size=32000, ln_type="rmsnorm", activation_type="swiglu", no_bias=True,
                    untie_embed=True, positional_embedding={"type": "rope"}),
    "qwen1p5b": dict(d_model=1536, num_attention_heads=12, num_attention_groups=2, head_dim=128, d_ffn=8960,
                     max_seq_len=768, vocab_size=151936, ln_type="rmsnorm", ln_eps=1e-6, activation_type="swiglu",
                     no_bias=True, qkv_bias=True, untie_embed=True, positional_embedding={"type": "rope", "base": 1e6}),
    "gpt2": dict(d_model=768, num_attention_heads=12, head_dim=64, d_ffn=3072, max_seq_len=1024,
                 max_position_embeddings=1024, vocab_size=50257),
}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="llama7b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--micro-batch", type=int, default=1)
    args = ap.parse_args(argv)
    from ironcore_b200.config import default_config, validate_config
    from ironcore_b200.ops import native
    from ironcore_b200.trainer import Trainer

    c = default_config()
    c.model(name="llama" if args.shape != "gpt2" else "gpt2", num_layers=args.layers, precision="bf16", dropout_embd=0.0,
            dropout_attn=0.0, dropout_mlp=0.0, reset_position_ids=False, reset_attention_mask=False, **SHAPES[args.shape])
    c.data(task_type="synthetic", vocab_size=SHAPES[args.shape]["vocab_size"])
    c.trainer(micro_batch_size=args.micro_batch, train_batch_size=args.micro_batch * args.iters,
              gradient_accumulation_steps=None, log_interval=10 ** 9)
    c.operation(train_steps=2, no_save=True)
    c.parallel(world_size=1, rank=0)
    c.utils(report_memory_usage=False)
    validate_config(c)
    tr = Trainer(c)
    tr.train_step(0)
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push("profiled_step")
    loss, _, _ = tr.train_step(1)
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    native.check_status()
    print(f"profile_step ok: loss {float(loss):.4f}, native calls {native.launches()}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
