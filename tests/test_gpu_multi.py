"""Fused compute+collective kernels on 2 GPUs against the NCCL + GEMM composition.
Skipped when fewer than two CUDA devices are visible."""

import os

import pytest
import torch

from helpers import free_port

pytestmark = pytest.mark.gpu


def _need_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")


def _worlds():
    """Rank counts to run the raw-kernel checks at: 2, and 4 / 8 when the box has them (the NVSwitch
    multicast forms are the default from 4 ranks up)."""
    n = torch.cuda.device_count()
    return sorted({2, max(w for w in (2, 4, 8) if w <= n)})


def _worker(rank, world, port, fn_name, out_q):
    import traceback

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        globals()[fn_name](rank, world)
        torch.cuda.synchronize()
        from ironcore_b200.ops import native

        native.check_status()
        dist.barrier()
        dist.destroy_process_group()
        out_q.put((rank, "ok"))
    except Exception:
        out_q.put((rank, traceback.format_exc()))


def _spawn(fn_name, world=2):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
    results = []
    while not q.empty():
        results.append(q.get())
    bad = [r for r in results if r[1] != "ok"]
    for p in procs:
        if p.is_alive():
            p.terminate()
            bad.append((-1, "timeout"))
    assert not bad and len(results) == world, "\n".join(f"[rank {r}] {m}" for r, m in bad)


def _close(a, b, k):
    # bf16 rounding of the inputs' products plus up to two output roundings (one of them inside the
    # switch when the reduction runs through the multicast address): 1 ulp = 2^-7 relative.
    err = (a.float() - b.float()).abs().max().item()
    assert err <= 3e-2 * (k ** 0.5) + 2.0 ** -7 * b.float().abs().max().item(), err


def check_raw_kernels(rank, world):
    import torch.distributed as dist

    from ironcore_b200.parallel.fused_comm import FusedTP

    torch.manual_seed(100 + rank)
    tokens, d, n = 1024 * max(1, world // 2), 512, 768
    rows = tokens // world
    for it in range(6):   # several epochs: flags are cumulative, buffers alternate
        if it % 3 == 0:   # plain P2P form first, then the NVLS (multimem) form where the fabric has multicast
            ws = FusedTP(tokens, d, dist.group.WORLD, nvls=(it >= 3), num_slots=2)
        x = torch.randn(rows, d, device="cuda").bfloat16()
        w = torch.randn(d, n, device="cuda").bfloat16()
        dist.broadcast(w, 0)
        full = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        y = ws.ag_gemm(x, w, a_major=0, b_major=1, n=n)
        _close(y, full.float() @ w.float(), d)
        # wgrad form: gathered^T @ dy
        dy = torch.randn(tokens, n, device="cuda").bfloat16()
        dw = ws.ag_gemm(x, dy, a_major=1, b_major=1, n=n)
        _close(dw, full.float().t() @ dy.float(), tokens)
        # GEMM -> reduce-scatter with bias and residual
        a = torch.randn(tokens, 384, device="cuda").bfloat16()
        b = torch.randn(384, d, device="cuda").bfloat16()
        bias = torch.randn(d, device="cuda").bfloat16()
        res = torch.randn(rows, d, device="cuda").bfloat16()
        out = ws.gemm_rs(a, b, b_major=1, bias=bias, residual=res)
        part = (a.float() @ b.float()).contiguous()
        ref = torch.empty(rows, d, device="cuda")
        dist.reduce_scatter_tensor(ref, part)
        _close(out, ref + bias.float() + res.float(), 384 * world)
        # GEMM -> reduce-scatter -> RMSNorm -> gather into a slot, consumed by a gather GEMM that only waits
        gamma = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
        dist.broadcast(gamma, 0)
        slot = ws.slots[it % 2]
        h, rstd = ws.gemm_rs(a, b, b_major=1, bias=bias, residual=res, norm=(gamma, 1e-5, 0.0, slot))
        y2 = ws.ag_gemm(slot.local, w, a_major=0, b_major=1, n=n, slot=slot, pushed=True)
        _close(h, ref + bias.float() + res.float(), 384 * world)
        hf = h.float()
        normed = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()).bfloat16()
        assert torch.allclose(rstd, torch.rsqrt(hf.pow(2).mean(-1) + 1e-5), rtol=1e-4, atol=1e-6)
        full_n = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full_n, normed)
        torch.cuda.synchronize()
        dist.barrier()
        assert (slot.buf.float() - full_n.float()).abs().max().item() <= 2.0 ** -6 * full_n.float().abs().max().item()
        _close(y2, full_n.float() @ w.float(), d)
        # the mirrored backward kernel: reduce-scatter -> RMSNorm backward (+ residual gradient) -> gather into
        # the scratch buffer of the next (pushed) gather GEMM
        from ironcore_b200.ops import kernels

        xin = torch.randn(rows, d, device="cuda").bfloat16()
        _, _, _, rstd_x = kernels.norm_fwd(xin, gamma, None, 1e-5, True)
        dres = torch.randn(rows, d, device="cuda").bfloat16()
        dx, dn = ws.gemm_rs_norm_bwd(a, b, b_major=1, residual=dres, gamma=gamma, w_offset=0.0, rstd=rstd_x, x=xin)
        wt = torch.randn(n, d, device="cuda").bfloat16()
        dist.broadcast(wt, 0)
        y3 = ws.ag_gemm(dx, wt, a_major=0, b_major=0, n=n, pushed=True)
        dn_ref = ref.bfloat16()
        _close(dn, ref, 384 * world)
        dx_ref, _, _ = kernels.norm_bwd(dn, xin, gamma, None, rstd_x, True, False, dres_in=dres)
        assert (dx.float() - dx_ref.float()).abs().max().item() <= 2.0 ** -6 * max(1.0, dx_ref.float().abs().max().item())
        full_dx = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full_dx, dx)
        assert torch.equal(ws.last_gathered, full_dx)
        _close(y3, full_dx.float() @ wt.float().t(), d)
        del dn_ref


def check_tp2_model_fused_matches_nccl(rank, world):
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer
    from helpers import tiny_config

    def run(fused, graph=False, norm_gather="on"):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama", d_model=256, d_ffn=512, num_layers=3, num_attention_heads=4, head_dim=64,
                          max_seq_len=256, max_position_embeddings=256, precision="bf16", vocab_size=1024)
        cfg.data.vocab_size = 1024
        cfg.model(reset_position_ids=False, reset_attention_mask=False)
        cfg.trainer(micro_batch_size=2, train_batch_size=8 if graph else 2, gradient_accumulation_steps=None,
                    tensor_model_parallel_size=world, cuda_graph=graph)
        cfg.parallel(world_size=world, rank=rank, local_rank=rank, sequence_parallel=True, fused_comm=fused,
                     fused_norm_gather=norm_gather)
        cfg.operation.train_steps = 3
        validate_config(cfg)
        tr = Trainer(cfg)
        if fused:
            assert any(hasattr(getattr(m, "fused", None), "g_epoch") for m in tr.model.modules())
            linked = sum(int(l.fuse_norm_gather) for l in tr.model.model.layers)
            assert linked == (3 if norm_gather == "on" else 0), linked
        return [float(tr.train_step(s)[0]) for s in range(3)]

    a = run(False)
    b = run(True)
    for x, y in zip(a, b):
        assert abs(x - y) < 5e-2, (a, b)
    c = run(True, norm_gather="off")      # fused GEMM+collective kernels, separate norm kernels
    for x, y in zip(a, c):
        assert abs(x - y) < 5e-2, (a, c)
    # CUDA-graph replay of the micro-batch with the fused kernels inside (4 micro-batches per step)
    graphed = run(True, graph=True)
    assert all(l == l and l < 20 for l in graphed), graphed


def check_dp2_fused_zero_matches_nccl(rank, world):
    """Pure data parallelism with ZeRO-1: the two-kernel fused step (P2P gradient reduction, in-kernel norm
    exchange, Adam, P2P parameter broadcast) against reduce-scatter / all-reduce / all-gather on NCCL."""
    import os

    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer
    from helpers import tiny_config

    def run(fused, nvls="off"):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama", d_model=256, d_ffn=512, num_layers=2, num_attention_heads=4, head_dim=64,
                          max_seq_len=128, max_position_embeddings=128, precision="bf16", vocab_size=1024)
        cfg.data.vocab_size = 1024
        cfg.model(reset_position_ids=False, reset_attention_mask=False)
        cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None,
                    tensor_model_parallel_size=1)
        cfg.parallel(world_size=world, rank=rank, local_rank=rank, zero_stage=1, fused_comm=True, fused_zero=fused,
                     nvls=nvls)
        cfg.optim(max_lr=1e-3, clip_grad=0.5, weight_decay=0.1)
        cfg.operation.train_steps = 4
        validate_config(cfg)
        tr = Trainer(cfg)
        assert (tr.optimizer.fused_zero is not None and tr.optimizer.fused_zero.ready) == fused
        out = [tr.train_step(s) for s in range(4)]
        losses = [float(o[0]) for o in out]
        norms = [float(o[1]) for o in out]
        flat = tr.optimizer.groups[0].param_buf.float().clone()
        return losses, norms, flat

    la, na, pa = run(False)
    for nvls in ("off", "on"):
        lb, nb, pb = run(True, nvls)
        for x, y in zip(la, lb):
            assert abs(x - y) < 2e-2, (la, lb)
        for x, y in zip(na, nb):
            assert abs(x - y) < 2e-2 * max(1.0, abs(x)), (na, nb)
        assert (pa - pb).abs().max().item() < 2e-2, (pa - pb).abs().max().item()


def check_ep2_fused_moe_matches_nccl(rank, world):
    """Expert parallelism over 2 GPUs: dispatch / combine inside kernels (P2P stores and loads into the
    grouped GEMM's layout) against the all-to-all composition, block level (output and gradients) and
    three trainer steps."""
    import os

    import torch.distributed as dist

    from ironcore_b200.config import validate_config
    from ironcore_b200.models.moe import MoEBlock
    from ironcore_b200.parallel import mesh
    from ironcore_b200.parallel.fused_moe import release_workspaces
    from ironcore_b200.trainer import Trainer
    from helpers import tiny_config

    def cfg_for():
        cfg = tiny_config("llama", d_model=256, d_ffn=512, num_layers=2, num_attention_heads=4, head_dim=64,
                          num_attention_groups=2, max_seq_len=128, max_position_embeddings=128, precision="bf16",
                          vocab_size=1024)
        cfg.data.vocab_size = 1024
        cfg.model(reset_position_ids=False, reset_attention_mask=False)
        cfg.model.moe(num_experts=8, top_k=2, expert_d_ffn=128, num_shared_experts=1, aux_loss_coeff=0.01)
        cfg.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None,
                    tensor_model_parallel_size=1)
        cfg.parallel(world_size=world, rank=rank, local_rank=rank, expert_model_parallel_size=world)
        cfg.operation.train_steps = 3
        validate_config(cfg)
        return cfg

    def block_run(fused):
        from ironcore_b200.parallel.symmetric import POLICY

        POLICY.fused_moe = fused
        release_workspaces()
        mesh.destroy_model_parallel()
        cfg = cfg_for()
        mesh.initialize_model_parallel(1, world)
        torch.manual_seed(5)
        blk = MoEBlock(cfg, dtype=torch.bfloat16, device=torch.device("cuda"))
        for p in blk.parameters():
            torch.nn.init.normal_(p, std=0.05)
        torch.manual_seed(11 + rank)
        x = torch.randn(256, 256, device="cuda").bfloat16().requires_grad_(True)
        out, aux = blk(x)
        assert (blk.fused_ep is not None) == fused
        g = torch.randn_like(out)
        (out * g).sum().backward()
        return out.detach().float(), x.grad.float(), blk.experts_up.grad.float(), blk.router.weight.grad.float()

    a = block_run(False)
    b = block_run(True)
    for u, v, tol in zip(a, b, (3e-2, 3e-2, 1e-1, 1e-1)):
        assert (u - v).abs().max().item() <= tol * max(1.0, u.abs().max().item()), (u - v).abs().max().item()

    def train_run(fused):
        release_workspaces()
        mesh.destroy_model_parallel()
        cfg = cfg_for()
        cfg.parallel.fused_moe = fused
        tr = Trainer(cfg)
        return [float(tr.train_step(s)[0]) for s in range(3)]

    la, lb = train_run(False), train_run(True)
    for x, y in zip(la, lb):
        assert abs(x - y) < 5e-2, (la, lb)


def check_dp2_muon_sharded_state_matches_replicated(rank, world):
    """Muon under data parallelism: with the optimizer state sharded (ZeRO-1) the matrix owners must still see
    whole, fully reduced gradient matrices; the run has to match the replicated-state run."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer
    from helpers import tiny_config

    def run(zero):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama", d_model=256, d_ffn=512, num_layers=2, num_attention_heads=4, head_dim=64,
                          max_seq_len=128, max_position_embeddings=128, precision="bf16", vocab_size=1024)
        cfg.data.vocab_size = 1024
        cfg.model(reset_position_ids=False, reset_attention_mask=False)
        cfg.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None,
                    tensor_model_parallel_size=1)
        cfg.parallel(world_size=world, rank=rank, local_rank=rank, zero_stage=zero)
        cfg.optim(optimizer="muon", muon_lr=0.02, max_lr=1e-3, clip_grad=1.0)
        cfg.operation.train_steps = 3
        validate_config(cfg)
        tr = Trainer(cfg)
        losses = [float(tr.train_step(s)[0]) for s in range(3)]
        return losses, tr.optimizer.groups[0].param_buf.float().clone()

    la, pa = run(0)
    lb, pb = run(1)
    for x, y in zip(la, lb):
        assert abs(x - y) < 2e-2, (la, lb)
    assert (pa - pb).abs().max().item() < 2e-2, (pa - pb).abs().max().item()


def check_fsdp2_matches_dp2(rank, world):
    """Full-shard FSDP on 2 GPUs (asynchronous parameter gathers and gradient reduce-scatters) against the
    replicated data-parallel run, with Adam and with Muon."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.ops import native
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer
    from helpers import tiny_config

    def run(fsdp, optimizer, fused_gather=False):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama", d_model=256, d_ffn=512, num_layers=3, num_attention_heads=4, head_dim=64,
                          max_seq_len=128, max_position_embeddings=128, precision="bf16", vocab_size=1024)
        cfg.data.vocab_size = 1024
        cfg.model(reset_position_ids=False, reset_attention_mask=False)
        cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None,
                    tensor_model_parallel_size=1)
        cfg.parallel(world_size=world, rank=rank, local_rank=rank, use_fsdp=fsdp, fsdp_mixed_precision="mixed",
                     fsdp_fused_gather=fused_gather)
        cfg.optim(optimizer=optimizer, muon_lr=0.02, max_lr=1e-3, clip_grad=1.0)
        cfg.operation.train_steps = 3
        validate_config(cfg)
        tr = Trainer(cfg)
        if fused_gather:
            assert tr.model.pool is not None, "the in-kernel gather was asked for and must be in use"
        losses = [float(tr.train_step(s)[0]) for s in range(3)]
        sd = {k: v.float().clone() for k, v in tr.model.canonical_state_dict().items()}
        losses.append(float(tr.train_step(3)[0]))         # and on after a state dict went through private buffers
        native.check_status()
        return losses, sd

    for optimizer in ("adam", "muon"):
        la, sa = run(False, optimizer)
        for fused_gather in (False, True):
            lb, sb = run(True, optimizer, fused_gather)
            for x, y in zip(la, lb):
                assert abs(x - y) < 3e-2, (optimizer, fused_gather, la, lb)
            worst = max((sa[k] - sb[k]).abs().max().item() for k in sa)
            assert worst < 3e-2, (optimizer, fused_gather, worst)


def check_fsdp_comm_kernels(rank, world):
    """Parameter gather and gradient reduce-scatter kernels over symmetric memory against NCCL."""
    import torch.distributed as dist

    from ironcore_b200.parallel.fsdp_comm import FsdpCommPool

    torch.manual_seed(50 + rank)
    n = 8 * world * 4096
    for reduce_dtype in (torch.float32, torch.bfloat16):
        pool = FsdpCommPool(dist.group.WORLD, n, torch.bfloat16, reduce_dtype)
        for it in range(3):
            slot = it % 2
            shard = torch.randn(n // world, device="cuda").bfloat16()
            ref = torch.empty(n, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(ref, shard)
            full = pool.gather(shard, slot)
            torch.cuda.synchronize()
            assert torch.equal(full, ref)
            flat = torch.randn(n, device="cuda").to(reduce_dtype)
            pool.flat_view(slot, n).copy_(flat)
            acc = torch.ones(n // world, device="cuda")
            pool.reduce_scatter(slot, acc, 0.5)
            want = torch.empty(n // world, device="cuda")
            dist.reduce_scatter_tensor(want, flat.float())
            torch.cuda.synchronize()
            assert (acc - (1.0 + 0.5 * want)).abs().max().item() < 2e-2


def check_dp2_overlapped_reduction_matches_whole_buffer(rank, world):
    """ZeRO-1 over two ranks with two micro-batches per step: gradient buckets all-reduced behind the last
    backward pass against one reduce-scatter of the whole buffer inside the step (both on NCCL)."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer
    from helpers import tiny_config

    def run(overlap):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama", d_model=256, d_ffn=512, num_layers=2, num_attention_heads=4, head_dim=64,
                          max_seq_len=128, max_position_embeddings=128, precision="bf16", vocab_size=1024)
        cfg.data.vocab_size = 1024
        cfg.model(reset_position_ids=False, reset_attention_mask=False)
        cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None,
                    tensor_model_parallel_size=1, cuda_graph=False)
        cfg.parallel(world_size=world, rank=rank, local_rank=rank, zero_stage=1, fused_zero=False,
                     overlap_grad_reduce=overlap, grad_bucket_mb=1.0)
        cfg.optim(max_lr=1e-3, clip_grad=0.5, weight_decay=0.1)
        cfg.operation.train_steps = 3
        validate_config(cfg)
        tr = Trainer(cfg)
        assert tr.optimizer.fused_zero is None and tr.optimizer.overlap == overlap
        launched = []
        if overlap:
            real = tr.optimizer._launch_bucket
            tr.optimizer._launch_bucket = lambda gi, bi: (launched.append(tr.optimizer._overlap_active), real(gi, bi))
        out = [tr.train_step(s) for s in range(3)]
        if overlap:
            assert len(launched) == 3 * len(tr.optimizer.groups[0].buckets) > 3 and all(launched), launched
        return [float(o[0]) for o in out], [float(o[1]) for o in out], tr.optimizer.groups[0].param_buf.float().clone()

    la, na, pa = run(False)
    lb, nb, pb = run(True)
    for x, y in zip(la, lb):
        assert abs(x - y) < 2e-2, (la, lb)
    for x, y in zip(na, nb):
        assert abs(x - y) < 2e-2 * max(1.0, abs(x)), (na, nb)
    assert (pa - pb).abs().max().item() < 2e-2, (pa - pb).abs().max().item()


def test_fused_tp_kernels_two_gpus():
    _need_two()
    for world in _worlds():
        _spawn("check_raw_kernels", world)


def test_dp2_fused_zero_step_vs_nccl():
    _need_two()
    _spawn("check_dp2_fused_zero_matches_nccl")


def test_dp2_overlapped_bucket_reduction():
    _need_two()
    _spawn("check_dp2_overlapped_reduction_matches_whole_buffer")


def test_fsdp2_matches_dp2():
    _need_two()
    _spawn("check_fsdp2_matches_dp2")


def test_fsdp_comm_kernels_two_gpus():
    _need_two()
    _spawn("check_fsdp_comm_kernels")


def test_dp2_muon_sharded_state():
    _need_two()
    _spawn("check_dp2_muon_sharded_state_matches_replicated")


def test_ep2_fused_moe_vs_nccl():
    _need_two()
    _spawn("check_ep2_fused_moe_matches_nccl")


def test_tp2_sp_model_fused_vs_nccl():
    _need_two()
    _spawn("check_tp2_model_fused_matches_nccl")
