"""Muon through the trainer: the learning-rate schedule of the Muon group, and checkpoint / resume of the
momentum that lives on each matrix's owner rank (2 CPU ranks over Gloo)."""

import math

import pytest
import torch

from helpers import run_distributed, tiny_config


def _muon_config(**optim):
    cfg = tiny_config("llama")
    cfg.optim(optimizer="muon", muon_lr=0.02, max_lr=3e-4, min_lr=3e-5, warmup_steps=4, annealing_steps=10,
              lr_scheduler="cosine", **optim)
    cfg.operation.train_steps = 20
    return cfg


def test_muon_group_follows_the_schedule_scaled_once():
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = _muon_config()
    validate_config(cfg)
    tr = Trainer(cfg)
    groups = tr.optimizer.param_groups
    assert [g["name"] for g in groups] == ["adam", "muon"]
    ratio = 0.02 / 3e-4
    seen = []
    for t in range(1, 16):          # the scheduler holds lr(t) for optimizer step t (1-based)
        adam, muon = groups[0]["lr"], groups[1]["lr"]
        seen.append(muon)
        if t <= 4:
            want = 3e-4 * t / 4
        elif t >= 14:
            want = 3e-5
        else:
            want = 3e-5 + (3e-4 - 3e-5) * (1 + math.cos(math.pi * (t - 4) / 10)) / 2
        assert adam == pytest.approx(want, rel=1e-9)
        assert muon == pytest.approx(want * ratio, rel=1e-9)
        tr.lr_scheduler.step()
    assert max(seen) == pytest.approx(0.02, rel=1e-9)      # peak is muon_lr, not muon_lr * muon_lr / max_lr
    # a reloaded scheduler reproduces the same rates
    sd = tr.lr_scheduler.state_dict()
    tr2 = Trainer(cfg)
    tr2.lr_scheduler.load_state_dict(sd)
    assert tr2.optimizer.param_groups[1]["lr"] == pytest.approx(groups[1]["lr"], rel=1e-12)


def _resume_worker(rank, world, fsdp, ckpt_dir):
    from ironcore_b200.checkpoint import load_checkpoint, save_checkpoint
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    def make():
        cfg = _muon_config()
        cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None, model_path=ckpt_dir)
        cfg.parallel(world_size=world, rank=rank, use_fsdp=fsdp, fsdp_mixed_precision="fp32")
        cfg.model(hf_model_type="llama", hf_architecture="LlamaForCausalLM")
        validate_config(cfg)
        return cfg, Trainer(cfg)

    cfg, tr = make()
    for s in range(2):
        tr.train_step(s)
    save_checkpoint(cfg, tr.model, tr.optimizer, tr.lr_scheduler, 1)
    tr.train_step(2)
    want = {k: v.clone() for k, v in tr.model.canonical_state_dict().items()}
    accum = cfg.trainer.gradient_accumulation_steps
    mesh.destroy_model_parallel()

    cfg2, tr2 = make()
    last = load_checkpoint(cfg2, tr2.model, tr2.optimizer, tr2.lr_scheduler)
    assert last == 1
    for _ in range(2 * accum):          # the synthetic stream does not rewind: skip what was consumed
        next(tr2.data_iterator["train"])
    tr2.train_step(2)
    got = tr2.model.canonical_state_dict()
    for k in want:
        assert torch.equal(want[k], got[k]), f"rank {rank}: {k} differs after resume " \
                                             f"(max {float((want[k] - got[k]).abs().max()):.3e})"


@pytest.mark.parametrize("fsdp", [False, True])
def test_muon_momentum_survives_resume_on_two_ranks(tmp_path, fsdp):
    run_distributed(_resume_worker, 2, fsdp, str(tmp_path / "ckpt"))


def _mesh_worker(rank, world, tp, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = _muon_config(muon_weight_decay=0.01)
    cfg.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None,
                tensor_model_parallel_size=tp)
    cfg.parallel(world_size=world, rank=rank, zero_stage=1, sequence_parallel=tp > 1)
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(3)]
    merged = merge_model_parallel_state(dict(tr.model.canonical_state_dict()), tr.model.canonical_shard_info())
    if rank == 0:
        torch.save({"losses": losses, "sd": merged}, out_path)


def test_muon_update_packs_on_tp_by_dp_mesh_match_dp(tmp_path):
    """Owners publish their matrices' updates through one all-gather of per-owner packs; on a TP2 x DP2 mesh the
    packs hold the tensor-parallel slices. Same data-parallel size, same data: the merged weights must agree.
    (DP2 itself is checked against the FSDP implementation of Muon in test_fsdp_cpu.)"""
    a, b = str(tmp_path / "dp2.pt"), str(tmp_path / "tp2dp2.pt")
    run_distributed(_mesh_worker, 2, 1, a)
    run_distributed(_mesh_worker, 4, 2, b)
    r0, r1 = torch.load(a), torch.load(b)
    assert r0["losses"] == pytest.approx(r1["losses"], abs=3e-4)
    for k, v in r0["sd"].items():
        assert torch.allclose(v, r1["sd"][k], atol=3e-4, rtol=1e-3), k
