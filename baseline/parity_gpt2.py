"""Loss-curve parity on CPU: GPT-2 pretraining in fp32, the unmodified reference (from
``baseline/_ref``, with the import-time shims of :mod:`baseline.reference_arm`) against
``ironcore_b200`` on the same initial weights, the same token batches and the same optimizer.

    python -m baseline.parity_gpt2 [--layers 12 --steps 20 --micro-batch 4 --accum 2 --seq 256]

Setup of both sides: pre-LayerNorm GPT-2 (d_model 768, 12 heads, FFN 3072 GELU, learned absolute
positions, vocab 50257, tied embeddings, init std 0.02), Adam beta (0.9, 0.95), lr 6e-4 with a
10-step warm-up then cosine decay, weight decay 0.1, gradient clipping 1.0, token ids uniform
from seed 1234. The reference model is built first; its ``state_dict`` is loaded into our model by
name (the parameter names are the shared checkpoint format), so both start from identical weights.
One intended difference: the reference takes the softmax over the padded vocabulary (50304 columns,
47 of them padding), ours masks the padding columns, so at vocab 50257 the curves differ by about
ln(50304/50257) = 9e-4 at initialisation; with a vocabulary that needs no padding they agree to 1e-6.
Prints one JSON line with both loss curves and the largest absolute difference.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _batches(vocab: int, micro_batch: int, seq: int, n: int, seed: int = 1234):
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for _ in range(n):
        tok = torch.randint(0, vocab, (micro_batch, seq + 1), generator=g)
        out.append({"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()})
    return out


def run_reference(args, batches):
    """Returns (loss curve, initial state dict) of the reference trainer, or raises."""
    import torch

    from baseline.reference_arm import REF_DIR, _install_shims

    if not os.path.isdir(os.path.join(REF_DIR, "ironcore")):
        raise FileNotFoundError("baseline/_ref is missing")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        import socket

        with socket.socket() as sock:
            sock.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(sock.getsockname()[1])
    os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1")
    gv, tr = _install_shims(args.vocab)
    from ironcore.config import (DataConfig, InitConfig, MainConfig, ModelConfig, OperationConfig, OptimConfig,
                                 ParallelConfig, TrainerConfig, UtilsConfig, _config_validation)
    from ironcore.training_utils import forward_step, loss_func

    cfg = MainConfig(model=ModelConfig(), init=InitConfig(), optim=OptimConfig(), data=DataConfig(),
                     parallel=ParallelConfig(), trainer=TrainerConfig(), operation=OperationConfig(),
                     utils=UtilsConfig())
    m = cfg.model
    m.name = "gpt2"
    m.d_model, m.d_ffn, m.num_layers = args.d_model, 4 * args.d_model, args.layers
    m.num_attention_heads = m.num_attention_groups = args.heads
    m.head_dim = args.d_model // args.heads
    m.max_seq_len = m.max_position_embeddings = args.seq
    m.dropout_embd = m.dropout_attn = m.dropout_mlp = 0.0
    m.precision = "float32"
    m.reset_position_ids = m.reset_attention_mask = False
    m.positional_embedding.type = "absolute"
    m.untie_embed = False
    m.no_bias = False
    m.ln_type = "layernorm"
    m.ln_eps = 1e-5
    m.activation_type = "gelu"
    cfg.data.vocab_size = args.vocab
    cfg.trainer.micro_batch_size = args.micro_batch
    cfg.trainer.train_batch_size = args.micro_batch * args.accum
    cfg.trainer.gradient_accumulation_steps = None
    cfg.trainer.tensor_model_parallel_size = 1
    cfg.trainer.vocab_padding_unit = args.vocab_padding_unit
    cfg.trainer.use_flash_attn = False
    cfg.trainer.model_path = ""
    cfg.trainer.log_interval = 10 ** 9
    cfg.operation.train_steps = args.total_steps
    cfg.operation.no_save = True
    cfg.optim.max_lr, cfg.optim.min_lr = 6e-4, 6e-5
    cfg.optim.lr_scheduler = "cosine"
    cfg.optim.warmup_steps = 10
    cfg.optim.annealing_steps = args.total_steps
    cfg.optim.adam_beta1, cfg.optim.adam_beta2 = 0.9, 0.95
    cfg.optim.weight_decay, cfg.optim.clip_grad = 0.1, 1.0
    cfg.init.init_std, cfg.init.seed = 0.02, 1234
    cfg.parallel.rank, cfg.parallel.world_size, cfg.parallel.local_rank = 0, 1, 0
    cfg.utils.report_memory_usage = False
    _config_validation(cfg)

    def cycle():
        i = 0
        while True:
            yield batches[i % len(batches)]
            i += 1

    iters = {"train": cycle(), "eval": None, "test": None}
    tr.get_data_iterator = lambda config: iters
    gv.GLOBAL_STATES = None
    trainer = tr.Trainer(cfg, forward_step, loss_func)
    model = trainer.model.module if hasattr(trainer.model, "module") else trainer.model
    init_state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    losses = []
    for s in range(args.steps):
        loss, _, _ = trainer.train_step(s)
        losses.append(float(loss))
    sched = {k: getattr(cfg.optim, k, None) for k in ("lr_scheduler", "warmup_steps", "annealing_steps", "max_lr",
                                                      "min_lr")}
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()
    return losses, init_state, sched


def run_ours(args, batches, init_state=None):
    import torch

    from ironcore_b200.config import default_config, validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    mesh.destroy_model_parallel()
    c = default_config()
    c.model(name="gpt2", d_model=args.d_model, d_ffn=4 * args.d_model, num_layers=args.layers,
            num_attention_heads=args.heads, num_attention_groups=args.heads, head_dim=args.d_model // args.heads,
            max_seq_len=args.seq, max_position_embeddings=args.seq, precision="fp32", vocab_size=args.vocab,
            dropout_embd=0.0, dropout_attn=0.0, dropout_mlp=0.0, untie_embed=False, no_bias=False,
            ln_type="layernorm", ln_eps=1e-5, activation_type="gelu", positional_embedding={"type": "absolute"},
            reset_position_ids=False, reset_attention_mask=False)
    c.data(task_type="synthetic", vocab_size=args.vocab)
    c.trainer(micro_batch_size=args.micro_batch, train_batch_size=args.micro_batch * args.accum,
              gradient_accumulation_steps=None, log_interval=10 ** 9, tensor_model_parallel_size=1,
              vocab_padding_unit=args.vocab_padding_unit)
    c.operation(train_steps=args.total_steps, no_save=True)
    c.optim(max_lr=6e-4, min_lr=6e-5, lr_scheduler="cosine", warmup_steps=10, annealing_steps=args.total_steps,
            adam_beta1=0.9, adam_beta2=0.95, weight_decay=0.1, clip_grad=1.0)
    c.init(init_std=0.02, seed=1234)
    c.parallel(world_size=1, rank=0, local_rank=0)
    c.utils(device="cpu") if hasattr(c.utils, "device") else None
    validate_config(c)
    trainer = Trainer(c)
    model = trainer.model.module if hasattr(trainer.model, "module") else trainer.model
    missing = unexpected = None
    if init_state is not None:
        own = model.canonical_state_dict()
        load = {k: v for k, v in init_state.items() if k in own and own[k].shape == v.shape}
        model.load_canonical_state_dict(load, strict=False)
        missing = [k for k in own if k not in load and not k.endswith(".theta")]
        unexpected = [k for k in init_state if k not in own]
        if hasattr(trainer.optimizer, "reload_model_params"):
            trainer.optimizer.reload_model_params()

    def cycle():
        i = 0
        while True:
            yield batches[i % len(batches)]
            i += 1

    trainer.data_iterator["train"] = cycle()
    losses = []
    for s in range(args.steps):
        loss, _, _ = trainer.train_step(s)
        losses.append(float(loss))
    trainer.finalize() if hasattr(trainer, "finalize") else None
    return losses, missing, unexpected


def compare(args):
    import torch

    torch.manual_seed(0)
    batches = _batches(args.vocab, args.micro_batch, args.seq, args.accum * args.steps)
    ref_losses, init_state, sched = run_reference(args, batches)
    our_losses, missing, unexpected = run_ours(args, batches, init_state)
    diffs = [abs(a - b) for a, b in zip(ref_losses, our_losses)]
    return {"reference_loss": ref_losses, "ironcore_b200_loss": our_losses, "max_abs_diff": max(diffs),
            "final_abs_diff": diffs[-1], "missing_in_ours": missing, "not_in_ours": unexpected,
            "reference_schedule": sched}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--d-model", dest="d_model", type=int, default=768)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--micro-batch", dest="micro_batch", type=int, default=4)
    ap.add_argument("--accum", type=int, default=2)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--total-steps", dest="total_steps", type=int, default=20)
    ap.add_argument("--vocab-padding-unit", dest="vocab_padding_unit", type=int, default=128,
                    help="1 = no padding columns, which removes the one intended difference between the two sides")
    args = ap.parse_args(argv)
    try:
        out = compare(args)
    except FileNotFoundError as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 0
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
