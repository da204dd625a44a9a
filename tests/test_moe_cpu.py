"""Mixture-of-experts block: dense restatement equivalence, padded layout, EP=2 == EP=1."""

import pytest
import torch

from helpers import run_distributed, tiny_config


def _moe_cfg(**kw):
    c = tiny_config("llama", num_attention_groups=4)
    c.model.moe(num_experts=8, top_k=2, expert_d_ffn=48, num_shared_experts=1, aux_loss_coeff=0.01)
    for k, v in kw.items():
        setattr(c.parallel, k, v)
    return c


def test_padded_layout_is_a_permutation_into_segments():
    from ironcore_b200.models.moe import padded_layout

    torch.manual_seed(0)
    ids = torch.randint(0, 5, (300,))
    dest, seg, tiles, counts = padded_layout(ids, 5, 300 + 5 * 127 + 1 + (128 - (300 + 5 * 127 + 1) % 128) % 128)
    assert dest.unique().numel() == 300
    for e in range(5):
        rows = dest[ids == e]
        assert rows.numel() == counts[e]
        if rows.numel():
            assert rows.min() >= seg[e] and rows.max() < seg[e + 1]
    assert int(seg[-1]) % 128 == 0
    used_tiles = int(seg[-1]) // 128
    assert (tiles[:used_tiles] >= 0).all() and (tiles[used_tiles:] == -1).all()


def test_moe_block_matches_dense_restatement():
    from ironcore_b200.config import validate_config
    from ironcore_b200.models.moe import MoEBlock, moe_reference
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = _moe_cfg()
    validate_config(cfg)
    torch.manual_seed(1)
    blk = MoEBlock(cfg, dtype=torch.float32)
    for p in blk.parameters():
        torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(37, 64, requires_grad=True)
    out, aux = blk(x)
    ref = moe_reference(x, blk.router.weight, blk.experts_up, blk.experts_down, 2, "swiglu") + blk.shared(x)
    assert torch.allclose(out, ref, atol=1e-5), (out - ref).abs().max()
    assert aux.item() > 0
    (out.sum() + aux).backward()
    assert blk.experts_up.grad is not None and blk.router.weight.grad is not None
    assert torch.isfinite(x.grad).all()


def _ep_worker(rank, world, ep, steps, out_path):
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = _moe_cfg(expert_model_parallel_size=ep)
    cfg.trainer(micro_batch_size=2, train_batch_size=2 * world, gradient_accumulation_steps=None)
    cfg.parallel(world_size=world, rank=rank)
    cfg.operation.train_steps = steps
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(steps)]
    from ironcore_b200.checkpoint.native import merge_model_parallel_state

    local = dict(tr.model.canonical_state_dict())
    names = {n for n in local if ".experts_" in n}
    merged = merge_model_parallel_state(local, tr.model.canonical_shard_info(), names)
    if rank == 0:
        torch.save({"losses": losses, "sd": merged}, out_path)


def test_ep2_matches_ep1(tmp_path):
    a, b = str(tmp_path / "ep1.pt"), str(tmp_path / "ep2.pt")
    run_distributed(_ep_worker, 2, 1, 3, a)
    run_distributed(_ep_worker, 2, 2, 3, b)
    r1, r2 = torch.load(a), torch.load(b)
    for x, y in zip(r1["losses"], r2["losses"]):
        assert abs(x - y) < 1e-4, (r1["losses"], r2["losses"])
    for k in r1["sd"]:
        assert torch.allclose(r1["sd"][k], r2["sd"][k], atol=1e-4, rtol=1e-3), k


def _tp_ep_worker(rank, world, tp, sp, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = _moe_cfg(expert_model_parallel_size=2)
    cfg.model.moe.aux_loss_coeff = 0.0     # (under sequence parallelism the balance loss is per token shard)
    cfg.trainer(micro_batch_size=2, train_batch_size=2 * (world // tp), gradient_accumulation_steps=None,
                tensor_model_parallel_size=tp)
    cfg.parallel(world_size=world, rank=rank, sequence_parallel=sp)
    cfg.operation.train_steps = 3
    validate_config(cfg)
    tr = Trainer(cfg)
    out = [tr.train_step(s) for s in range(3)]
    local = dict(tr.model.canonical_state_dict())
    merged = merge_model_parallel_state(local, tr.model.canonical_shard_info(), {n for n in local if ".experts_" in n})
    if rank == 0:
        torch.save({"losses": [float(o[0]) for o in out], "norms": [float(o[1]) for o in out], "sd": merged}, out_path)


@pytest.mark.parametrize("sp", [False, True])
def test_tensor_parallel_times_expert_parallel_matches_expert_parallel(tmp_path, sp):
    """TP2 x EP2 on four ranks against EP2 on two: the expert weights are copies on the tensor-parallel ranks, so
    under sequence parallelism (each rank routes its token shard) their gradients are summed over the group, and
    the gradient norm counts them once."""
    a, b = str(tmp_path / "ep2.pt"), str(tmp_path / "tp2ep2.pt")
    run_distributed(_tp_ep_worker, 2, 1, False, a)
    run_distributed(_tp_ep_worker, 4, 2, sp, b)
    r1, r2 = torch.load(a), torch.load(b)
    assert r1["losses"] == pytest.approx(r2["losses"], abs=2e-5)
    assert r1["norms"] == pytest.approx(r2["norms"], rel=1e-4)
    for k in r1["sd"]:
        assert torch.allclose(r1["sd"][k], r2["sd"][k], atol=1e-4, rtol=1e-3), k
