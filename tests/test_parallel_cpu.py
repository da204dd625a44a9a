"""Multi-rank host logic on CPU ranks over Gloo: mesh layout, TP / SP equivalence with the
single-rank model, ZeRO-1 equivalence with the replicated optimizer, universal checkpoints
across TP sizes."""

import os

import pytest
import torch

from helpers import run_distributed, tiny_config


def test_mesh_layout_matches_documented_example():
    from ironcore_b200.parallel.mesh import mesh_layout

    lay = mesh_layout(16, 4)
    assert lay["tp"][0] == [0, 1, 2, 3] and lay["tp"][3] == [12, 13, 14, 15]
    assert lay["dp"][0] == [0, 4, 8, 12] and lay["dp"][1] == [1, 5, 9, 13]
    lay = mesh_layout(8, 1, ep=4)
    assert lay["ep"] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert lay["edp"] == [[0, 4], [1, 5], [2, 6], [3, 7]]


# architecture switches of the families that ``tiny_config`` does not know by itself
_FAMILY_KW = {
    "phi2": dict(activation_type="gelu_new", untie_embed=True, positional_embedding={"type": "rope", "rotary_fraction": 0.5}),
    "gemma1": dict(no_bias=True, ln_type="rmsnorm", activation_type="geglu", untie_embed=False, num_attention_groups=2,
                   positional_embedding={"type": "rope"}),
}


def _reference_run(family, steps, accum=1):
    """Single-process TP=1 run: returns losses and the final canonical state dict."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    mesh.destroy_model_parallel()
    cfg = tiny_config(family, **_FAMILY_KW.get(family, {}))
    cfg.trainer(micro_batch_size=2, train_batch_size=2 * accum, gradient_accumulation_steps=None)
    cfg.operation.train_steps = steps
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(steps)]
    sd = {k: v.clone() for k, v in tr.model.canonical_state_dict().items()}
    return losses, sd


def _tp_worker(rank, world, family, sp, steps, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config(family, **_FAMILY_KW.get(family, {}))
    cfg.trainer(micro_batch_size=2, train_batch_size=2, gradient_accumulation_steps=None,
                tensor_model_parallel_size=world)
    cfg.parallel(world_size=world, rank=rank, sequence_parallel=sp)
    cfg.operation.train_steps = steps
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(steps)]
    merged = merge_model_parallel_state(dict(tr.model.canonical_state_dict()), tr.model.canonical_shard_info())
    if rank == 0:
        torch.save({"losses": losses, "sd": merged}, out_path)


@pytest.mark.parametrize("family,sp", [("gpt2", False), ("llama", False), ("llama", True), ("gpt2", True),
                                       ("qwen", True), ("phi2", True), ("gemma1", True)])
def test_tp2_matches_tp1(tmp_path, family, sp):
    steps = 3
    ref_losses, ref_sd = _reference_run(family, steps)
    out = str(tmp_path / "tp.pt")
    run_distributed(_tp_worker, 2, family, sp, steps, out)
    got = torch.load(out)
    for a, b in zip(ref_losses, got["losses"]):
        assert abs(a - b) < 2e-4, (ref_losses, got["losses"])
    for k, v in ref_sd.items():
        assert torch.allclose(v, got["sd"][k], atol=2e-4, rtol=1e-3), k


def _full_load_worker(rank, world, family, path):
    from ironcore_b200.config import validate_config
    from ironcore_b200.models.language_model import LanguageModel
    from ironcore_b200.parallel import mesh

    saved = torch.load(path)
    cfg = tiny_config(family, **_FAMILY_KW.get(family, {}))
    cfg.trainer(tensor_model_parallel_size=world)
    cfg.parallel(world_size=world, rank=rank)
    cfg.init.seed = 99          # different weights until the state dict is loaded
    validate_config(cfg)
    mesh.initialize_model_parallel(world)
    model = LanguageModel(cfg)
    model.load_state_dict(saved["sd"])
    with torch.no_grad():
        loss = float(model(saved["ids"], saved["labels"]))
    assert abs(loss - saved["loss"]) < 1e-4, (loss, saved["loss"])


@pytest.mark.parametrize("family", ["gpt2", "llama"])
def test_single_rank_state_dict_loads_into_tp2(tmp_path, family):
    """``load_state_dict`` slices unsharded tensors: a TP=1 ``state_dict()`` drives a TP=2 model to the same loss."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.models.language_model import LanguageModel
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = tiny_config(family, **_FAMILY_KW.get(family, {}))
    validate_config(cfg)
    mesh.initialize_model_parallel(1)
    model = LanguageModel(cfg)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 512, (2, 32), generator=g)
    labels = torch.randint(0, 512, (2, 32), generator=g)
    with torch.no_grad():
        loss = float(model(ids, labels))
    path = str(tmp_path / "full.pt")
    torch.save({"sd": model.state_dict(), "ids": ids, "labels": labels, "loss": loss}, path)
    mesh.destroy_model_parallel()
    run_distributed(_full_load_worker, 2, family, path)


def _zero_worker(rank, world, zero, steps, out_path, overlap=False, accum=1):
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config("llama")
    cfg.trainer(micro_batch_size=2, train_batch_size=4 * accum, gradient_accumulation_steps=None)
    cfg.parallel(world_size=world, rank=rank, zero_stage=zero, overlap_grad_reduce=overlap, grad_bucket_mb=0.05)
    cfg.operation.train_steps = steps
    validate_config(cfg)
    tr = Trainer(cfg)
    if overlap:
        launched = []
        real = tr.optimizer._launch_bucket
        tr.optimizer._launch_bucket = lambda gi, bi: (launched.append((gi, bi, tr.optimizer._overlap_active)), real(gi, bi))
    losses = [float(tr.train_step(s)[0]) for s in range(steps)]
    if overlap:
        nb = len(tr.optimizer.groups[0].buckets)
        # every bucket once per step, and all of them from inside the backward pass
        assert nb > 2 and len(launched) == nb * steps and all(active for _, _, active in launched), (nb, launched)
    sd = {k: v.clone() for k, v in tr.model.canonical_state_dict().items()}
    opt = tr.optimizer.state_dict()
    if rank == 0:
        torch.save({"losses": losses, "sd": sd, "opt": opt["state"]}, out_path)


def test_zero1_matches_replicated_optimizer(tmp_path):
    a, b = str(tmp_path / "z0.pt"), str(tmp_path / "z1.pt")
    run_distributed(_zero_worker, 2, 0, 3, a)
    run_distributed(_zero_worker, 2, 1, 3, b)
    r0, r1 = torch.load(a), torch.load(b)
    for k in r0["sd"]:
        assert torch.allclose(r0["sd"][k], r1["sd"][k], atol=1e-6), k
    for k in r0["opt"]:
        assert torch.allclose(r0["opt"][k]["exp_avg"], r1["opt"][k]["exp_avg"], atol=1e-7), k


@pytest.mark.parametrize("zero", [0, 1])
def test_overlapped_bucket_reduction_matches_whole_buffer_reduction(tmp_path, zero):
    a, b = str(tmp_path / "plain.pt"), str(tmp_path / "overlap.pt")
    run_distributed(_zero_worker, 2, zero, 3, a, False, 2)
    run_distributed(_zero_worker, 2, zero, 3, b, True, 2)
    r0, r1 = torch.load(a), torch.load(b)
    assert r0["losses"] == pytest.approx(r1["losses"], abs=1e-6)
    for k in r0["sd"]:
        assert torch.allclose(r0["sd"][k], r1["sd"][k], atol=1e-6), k


def _tp_dp_worker(rank, world, overlap, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config("llama")
    cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None, tensor_model_parallel_size=2)
    cfg.parallel(world_size=world, rank=rank, sequence_parallel=True, zero_stage=1, overlap_grad_reduce=overlap,
                 grad_bucket_mb=0.02)
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(2)]
    merged = merge_model_parallel_state(dict(tr.model.canonical_state_dict()), tr.model.canonical_shard_info())
    if rank == 0:
        torch.save({"losses": losses, "sd": merged}, out_path)


def test_overlapped_reduction_on_a_tp_by_dp_mesh(tmp_path):
    """TP2 x DP2 with sequence parallelism: the bucket all-reduces over the data-parallel group and the
    tensor-parallel sum of the replicated parameters' gradients commute."""
    a, b = str(tmp_path / "plain.pt"), str(tmp_path / "overlap.pt")
    run_distributed(_tp_dp_worker, 4, False, a)
    run_distributed(_tp_dp_worker, 4, True, b)
    r0, r1 = torch.load(a), torch.load(b)
    assert r0["losses"] == pytest.approx(r1["losses"], abs=1e-6)
    for k in r0["sd"]:
        assert torch.allclose(r0["sd"][k], r1["sd"][k], atol=1e-6), k


def _ckpt_save_worker(rank, world, path):
    from ironcore_b200.checkpoint import save_checkpoint
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config("llama")
    cfg.trainer(micro_batch_size=2, train_batch_size=2, gradient_accumulation_steps=None,
                tensor_model_parallel_size=world, model_path=path)
    cfg.parallel(world_size=world, rank=rank, sequence_parallel=True)
    cfg.operation.train_steps = 2
    validate_config(cfg)
    tr = Trainer(cfg)
    for s in range(2):
        tr.train_step(s)
    save_checkpoint(cfg, tr.model, tr.optimizer, tr.lr_scheduler, 1)


def test_universal_checkpoint_tp2_to_tp1(tmp_path):
    from ironcore_b200.checkpoint import load_checkpoint
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    path = str(tmp_path / "ck")
    run_distributed(_ckpt_save_worker, 2, path)
    ref_losses, ref_sd = _reference_run("llama", 2)
    mesh.destroy_model_parallel()
    cfg = tiny_config("llama")
    cfg.trainer(micro_batch_size=2, train_batch_size=2, gradient_accumulation_steps=None, model_path=path)
    cfg.operation.train_steps = 2
    validate_config(cfg)
    tr = Trainer(cfg)
    assert load_checkpoint(cfg, tr.model, tr.optimizer, tr.lr_scheduler) == 1
    for k, v in tr.model.canonical_state_dict().items():
        assert torch.allclose(v, ref_sd[k], atol=2e-4, rtol=1e-3), k
    assert tr.optimizer.step_count == 2


_RESUME_LAYOUTS = {
    "zero1_dp2": dict(parallel=dict(zero_stage=1)),
    "tp2_sp": dict(tp=2, parallel=dict(sequence_parallel=True)),
    "tp2_sp_per_rank_files": dict(tp=2, parallel=dict(sequence_parallel=True), operation=dict(save_dist_ckpt=True)),
    "ep2_zero1": dict(moe=dict(num_experts=4, top_k=2, expert_d_ffn=32, num_shared_experts=1),
                      parallel=dict(expert_model_parallel_size=2, zero_stage=1)),
    "fsdp2": dict(parallel=dict(use_fsdp=True, fsdp_mixed_precision="fp32")),
}


def _resume_worker(rank, world, layout, root, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    spec = _RESUME_LAYOUTS[layout]

    def run(steps, path):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama")
        if spec.get("moe"):
            cfg.model.moe(**spec["moe"])
        tp = spec.get("tp", 1)
        cfg.trainer(micro_batch_size=2, train_batch_size=2 * (world // tp), gradient_accumulation_steps=None,
                    tensor_model_parallel_size=tp, model_path=path, save_checkpoint_steps=100)
        cfg.parallel(world_size=world, rank=rank, **spec.get("parallel", {}))
        cfg.optim(lr_scheduler="cosine", warmup_steps=1, annealing_steps=10, max_lr=1e-3)
        cfg.operation(train_steps=steps, **spec.get("operation", {}))
        validate_config(cfg)
        tr = Trainer(cfg)
        assert tr.train() == steps - 1
        local = dict(tr.model.canonical_state_dict())
        return merge_model_parallel_state(local, tr.model.canonical_shard_info(), {n for n in local if ".experts_" in n})

    whole = run(4, os.path.join(root, "a"))
    run(2, os.path.join(root, "b"))
    resumed = run(4, os.path.join(root, "b"))
    if rank == 0:
        torch.save(max((whole[k].float() - resumed[k].float()).abs().max().item() for k in whole), out_path)


@pytest.mark.parametrize("layout", sorted(_RESUME_LAYOUTS))
def test_interrupted_run_on_two_ranks_continues_as_if_uninterrupted(tmp_path, layout):
    """Save after two steps, start over with new objects, train to step four: bit-identical to four steps in one go
    for every parallel layout and checkpoint form."""
    out = str(tmp_path / "diff.pt")
    run_distributed(_resume_worker, 2, layout, str(tmp_path), out)
    assert torch.load(out) == 0.0


_MOE4 = dict(num_experts=4, top_k=2, expert_d_ffn=32, num_shared_experts=1)
_CROSS = {      # name: ((world, layout) that writes the checkpoint, (world, layout) that resumes it)
    "tp2_to_tp1": ((2, dict(tp=2, gb=2, parallel=dict(sequence_parallel=True))), (1, dict(gb=2))),
    "tp1_to_tp2": ((1, dict(gb=2)), (2, dict(tp=2, gb=2, parallel=dict(sequence_parallel=True)))),
    "ep2_to_ep1": ((2, dict(moe=True, gb=4, parallel=dict(expert_model_parallel_size=2))), (2, dict(moe=True, gb=4))),
    "fsdp_to_zero1": ((2, dict(gb=4, parallel=dict(use_fsdp=True, fsdp_mixed_precision="fp32"))),
                      (2, dict(gb=4, parallel=dict(zero_stage=1)))),
}


def _cross_worker(rank, world, spec, steps, path, out_path):
    from ironcore_b200.checkpoint.native import merge_model_parallel_state
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    # 500 entries: padded to 504 on one tensor-parallel rank and to 512 on two (unit 8 x TP size)
    cfg = tiny_config("llama", vocab_size=500)
    cfg.data.vocab_size = 500
    if spec.get("moe"):
        cfg.model.moe(**_MOE4)
    cfg.trainer(micro_batch_size=2, train_batch_size=spec["gb"], gradient_accumulation_steps=None,
                tensor_model_parallel_size=spec.get("tp", 1), model_path=path, save_checkpoint_steps=100)
    cfg.parallel(world_size=world, rank=rank, **spec.get("parallel", {}))
    cfg.optim(lr_scheduler="cosine", warmup_steps=1, annealing_steps=10, max_lr=1e-3)
    cfg.operation(train_steps=steps)
    validate_config(cfg)
    tr = Trainer(cfg)
    tr.train()
    local = dict(tr.model.canonical_state_dict())
    merged = merge_model_parallel_state(local, tr.model.canonical_shard_info(), {n for n in local if ".experts_" in n})
    if rank == 0 and out_path:
        torch.save(merged, out_path)


@pytest.mark.parametrize("case", sorted(_CROSS))
def test_checkpoint_resumes_under_another_layout(tmp_path, case):
    """A merged checkpoint (weights and optimizer state) written under one parallel layout continues under another
    as the uninterrupted run of that other layout would (same data-parallel size, so the same data)."""
    (wa, sa), (wb, sb) = _CROSS[case]
    whole, ck = str(tmp_path / "whole"), str(tmp_path / "ck")
    run_distributed(_cross_worker, wb, sb, 4, whole, str(tmp_path / "whole.pt"))
    run_distributed(_cross_worker, wa, sa, 2, ck, None)
    run_distributed(_cross_worker, wb, sb, 4, ck, str(tmp_path / "resumed.pt"))
    a, b = torch.load(str(tmp_path / "whole.pt")), torch.load(str(tmp_path / "resumed.pt"))
    for k in a:
        assert a[k].shape == b[k].shape and torch.allclose(a[k], b[k], atol=1e-5, rtol=1e-4), k
