"""FSDP full-shard (Adam and Muon) on 2 CPU ranks must reproduce the replicated data-parallel run."""

import pytest
import torch

from helpers import run_distributed, tiny_config


def _worker(rank, world, fsdp, optimizer, steps, out_path):
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config("llama")
    cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None)
    cfg.parallel(world_size=world, rank=rank, use_fsdp=fsdp, fsdp_mixed_precision="fp32")
    cfg.optim(optimizer=optimizer, muon_lr=0.02, max_lr=1e-3)
    cfg.operation.train_steps = steps
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(steps)]
    base = tr.model
    sd = base.canonical_state_dict()
    sd = {k: v.clone() for k, v in sd.items()}
    if rank == 0:
        torch.save({"losses": losses, "sd": sd}, out_path)


@pytest.mark.parametrize("optimizer", ["adam", "muon"])
def test_fsdp_matches_replicated_dp(tmp_path, optimizer):
    a, b = str(tmp_path / "dp.pt"), str(tmp_path / "fsdp.pt")
    run_distributed(_worker, 2, False, optimizer, 3, a)
    run_distributed(_worker, 2, True, optimizer, 3, b)
    r0, r1 = torch.load(a), torch.load(b)
    for x, y in zip(r0["losses"], r1["losses"]):
        assert abs(x - y) < 1e-4, (r0["losses"], r1["losses"])
    tol = 1e-5 if optimizer == "adam" else 2e-3
    for k in r0["sd"]:
        assert torch.allclose(r0["sd"][k], r1["sd"][k], atol=tol, rtol=1e-3), k


def test_newton_schulz_orthogonalises():
    from ironcore_b200.optim.muon import newton_schulz_reference

    torch.manual_seed(0)
    g = torch.randn(48, 96)
    x = newton_schulz_reference(g, steps=5, dtype=torch.float32)
    s = torch.linalg.svdvals(x)
    assert s.max() < 1.3 and s.min() > 0.5   # singular values pulled towards 1
    gt = torch.randn(96, 48)
    xt = newton_schulz_reference(gt, steps=5, dtype=torch.float32)
    assert xt.shape == gt.shape


def _tp_worker(rank, world, fsdp, sp, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config("llama")
    cfg.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None, tensor_model_parallel_size=2)
    cfg.parallel(world_size=world, rank=rank, use_fsdp=fsdp, fsdp_mixed_precision="fp32", sequence_parallel=sp)
    cfg.optim(max_lr=1e-3, clip_grad=0.5)          # (the clip is active: the norm enters the update)
    cfg.operation.train_steps = 3
    validate_config(cfg)
    tr = Trainer(cfg)
    out = [tr.train_step(s) for s in range(3)]
    merged = merge_model_parallel_state(dict(tr.model.canonical_state_dict()), tr.model.canonical_shard_info())
    pn = float(tr.optimizer.param_norm())
    if rank == 0:
        torch.save({"losses": [float(o[0]) for o in out], "norms": [float(o[1]) for o in out], "sd": merged,
                    "param_norm": pn}, out_path)


@pytest.mark.parametrize("sp", [False, True])
def test_fsdp_next_to_tensor_parallelism_matches_data_parallel(tmp_path, sp):
    """FSDP over the data-parallel group of a TP2 x DP2 mesh: the gradient norm sums the tensor-parallel shards and
    counts the copies once, and with sequence parallelism the copies' gradients are summed over the TP group."""
    a, b = str(tmp_path / "dp.pt"), str(tmp_path / "fsdp.pt")
    run_distributed(_tp_worker, 4, False, sp, a)
    run_distributed(_tp_worker, 4, True, sp, b)
    r0, r1 = torch.load(a), torch.load(b)
    assert r0["losses"] == pytest.approx(r1["losses"], abs=1e-4)
    assert r0["norms"] == pytest.approx(r1["norms"], rel=1e-4)
    assert r0["param_norm"] == pytest.approx(r1["param_norm"], rel=1e-5)
    for k in r0["sd"]:
        assert torch.allclose(r0["sd"][k], r1["sd"][k], atol=1e-5, rtol=1e-3), k


def test_layouts_the_shard_engine_does_not_serve_are_refused():
    from ironcore_b200.config import validate_config

    cfg = tiny_config("llama")
    cfg.model.moe(num_experts=4, top_k=2, expert_d_ffn=32)
    cfg.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None)
    cfg.parallel(world_size=2, rank=0, use_fsdp=True, expert_model_parallel_size=2)
    with pytest.raises(ValueError, match="zero_stage"):
        validate_config(cfg)
