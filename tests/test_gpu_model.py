"""Whole-model numerics on the GPU: the bf16 native path against the fp32 PyTorch path with the
same weights, and the flat-buffer optimizer against the per-parameter reference update."""

import pytest
import torch

from helpers import tiny_config

pytestmark = pytest.mark.gpu


def _cfg(family, precision, **kw):
    c = tiny_config(family, d_model=256, d_ffn=512, num_layers=2, num_attention_heads=4, head_dim=64, max_seq_len=256,
                    max_position_embeddings=256, precision=precision, vocab_size=1024, **kw)
    c.data.vocab_size = 1024
    from ironcore_b200.config import validate_config

    validate_config(c)
    return c


@pytest.mark.parametrize("family", ["gpt2", "llama"])
def test_native_model_matches_fp32_reference(family):
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.ops import native

    torch.manual_seed(0)
    ref = LanguageModel(_cfg(family, "fp32"))
    nat = LanguageModel(_cfg(family, "bf16"), device=torch.device("cuda")).cuda()
    nat.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
    ref.load_state_dict({k: v.float().cpu() for k, v in nat.state_dict().items()})
    ids = torch.randint(0, 1024, (2, 257))
    x, y = ids[:, :-1], ids[:, 1:]
    loss_ref = ref(x, y)
    loss_ref.backward()
    native.reset_launches()
    loss_nat = nat(x.cuda(), y.cuda())
    loss_nat.backward()
    torch.cuda.synchronize()
    native.check_status()
    assert native.launches() > 20
    assert abs(loss_ref.item() - loss_nat.item()) < 3e-2, (loss_ref.item(), loss_nat.item())
    gref = dict(ref.named_parameters())
    worst = 0.0
    for name, p in nat.named_parameters():
        g = p.grad
        assert g is not None, name
        r = gref[name].grad
        denom = r.abs().max().item() + 1e-6
        worst = max(worst, (g.float().cpu() - r).abs().max().item() / denom)
    assert worst < 8e-2, worst


def test_trainer_native_loss_falls_and_matches_cpu():
    from ironcore_b200.trainer import Trainer

    def run(precision, device_ok):
        cfg = _cfg("llama", precision)
        cfg.optim.max_lr = 2e-3
        tr = Trainer(cfg)
        if not device_ok:
            assert tr.device.type == "cuda"
        from ironcore_b200.data.synthetic import SyntheticTokenStream

        batch = next(SyntheticTokenStream(1024, 256, 2, seed=3, pin=False))

        def it():
            while True:
                yield batch

        tr.data_iterator = {"train": it(), "eval": None, "test": None}
        return [float(tr.train_step(s)[0]) for s in range(6)]

    losses = run("bf16", True)
    assert losses[-1] < losses[0] - 0.3, losses


def test_moe_block_native_matches_dense_restatement():
    from ironcore_b200.models.moe import MoEBlock, moe_reference
    from ironcore_b200.ops import native
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = _cfg("llama", "bf16")
    cfg.model.moe(num_experts=8, top_k=2, expert_d_ffn=256, num_shared_experts=1, aux_loss_coeff=0.01)
    torch.manual_seed(5)
    blk = MoEBlock(cfg, dtype=torch.bfloat16, device=torch.device("cuda"))
    for p in blk.parameters():
        torch.nn.init.normal_(p, std=0.05)
    x = (0.5 * torch.randn(700, 256, device="cuda")).bfloat16().requires_grad_(True)
    out, aux = blk(x)
    torch.cuda.synchronize()
    native.check_status()
    xf = x.detach().float().requires_grad_(True)
    up = blk.experts_up.detach().float().requires_grad_(True)
    down = blk.experts_down.detach().float().requires_grad_(True)
    ref = moe_reference(xf, blk.router.weight.float(), up, down, 2, "swiglu")
    shared = blk.shared(x.detach()).float()
    # tokens whose two best experts are a near tie may route differently in bf16 and fp32: compare the rest
    idx_native = blk.route(x.detach())[1].sort(-1).values
    idx_ref = torch.topk(torch.softmax((xf.detach() @ blk.router.weight.float().t()), -1), 2, -1)[1].sort(-1).values
    same = (idx_native == idx_ref).all(-1)
    assert same.float().mean().item() > 0.9
    assert (out.float() - (ref + shared)).abs()[same].max().item() < 5e-2
    dy = torch.randn_like(out) * same[:, None].to(out.dtype)
    out.backward(dy)
    ref.backward(dy.float())
    gu = blk.experts_up.grad.float()
    # the routing-mismatch tokens still contribute (with zero upstream gradient they add nothing)
    assert (gu - up.grad).abs().max().item() < 8e-2 * max(up.grad.abs().max().item(), 1.0)
    gd = blk.experts_down.grad.float()
    assert (gd - down.grad).abs().max().item() < 8e-2 * max(down.grad.abs().max().item(), 1.0)


def test_cuda_graph_micro_batch_matches_eager():
    from ironcore_b200.trainer import Trainer

    def run(graph):
        cfg = _cfg("llama", "bf16", reset_position_ids=False, reset_attention_mask=False)
        cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None, cuda_graph=graph)
        from ironcore_b200.config import validate_config

        validate_config(cfg)
        tr = Trainer(cfg)
        return [float(tr.train_step(s)[0]) for s in range(3)]

    a, b = run(False), run(True)
    assert b is not None
    for x, y in zip(a, b):
        assert abs(x - y) < 2e-2, (a, b)


def test_router_kernel_selects_valid_experts_for_nan_rows():
    """A diverged run feeds NaN logits to the router: the kernel must still name K experts in range for every
    token (the downstream kernels index tables with them) while the probabilities keep the NaN for the loss."""
    from ironcore_b200.models import moe  # noqa: F401  (registers the router entry points)
    from ironcore_b200.ops import native

    t, e, k = 64, 64, 6
    logits = torch.randn(t, e, device="cuda")
    logits[5] = float("nan")
    logits[17, 3] = float("nan")
    probs = torch.empty_like(logits)
    w = torch.empty(t, k, device="cuda")
    idx = torch.full((t, k), -7, dtype=torch.int32, device="cuda")
    counts = torch.zeros(e, dtype=torch.int32, device="cuda")
    psum = torch.zeros(e, device="cuda")
    native.call("icb_router_fwd", native.ptr(logits), t, e, k, 1, native.ptr(probs), native.ptr(w), native.ptr(idx),
                native.ptr(counts), native.ptr(psum), native.stream_ptr())
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0 and int(idx.max()) < e
    assert all(len(set(row.tolist())) == k for row in idx.cpu())
    assert int(counts.sum()) == t * k
    assert torch.isnan(probs[5]).all() and torch.isfinite(probs[0]).all()


@pytest.mark.parametrize("experts,top_k,normalize", [(64, 6, False), (8, 2, True), (16, 1, False)])
def test_router_kernel_matches_eager(experts, top_k, normalize):
    """Router kernels (GEMM logits -> softmax / top-k / histogram / aux loss, and the backward) against the same
    computation in fp32 PyTorch on the logits the kernel saw."""
    from ironcore_b200.models.moe import _Router
    from ironcore_b200.ops import kernels, native

    torch.manual_seed(21)
    t, d, coeff = 1000, 256, 0.01
    x = torch.randn(t, d, device="cuda").bfloat16().requires_grad_(True)
    wr = (torch.randn(experts, d, device="cuda") * 0.3).bfloat16().requires_grad_(True)
    w, idx, aux = _Router.apply(x, wr, top_k, normalize, coeff)
    gw = torch.randn_like(w)
    ((w * gw).sum() + 3.0 * aux).backward()
    torch.cuda.synchronize()
    native.check_status()
    # reference from the same fp32 logits
    logits = kernels.mm_nt(x.detach(), wr.detach(), out_dtype=torch.float32).requires_grad_(True)
    probs = torch.softmax(logits, -1)
    rw, ridx = torch.topk(probs, top_k, -1)
    if normalize:
        rw = rw / rw.sum(-1, keepdim=True)
    f = torch.bincount(ridx.reshape(-1), minlength=experts).float() / (t * top_k)
    raux = coeff * experts * (f * probs.mean(0)).sum()
    assert torch.equal(idx.sort(-1).values, ridx.sort(-1).values)
    order = idx.argsort(-1)
    rorder = ridx.argsort(-1)
    assert torch.allclose(w.gather(-1, order), rw.gather(-1, rorder), atol=1e-6, rtol=1e-5)
    assert torch.allclose(aux, raux, rtol=1e-4, atol=1e-8)
    rgw = torch.zeros_like(rw).scatter(-1, rorder, gw.gather(-1, order))   # same upstream gradient per expert
    ((rw * rgw).sum() + 3.0 * raux).backward()
    dl = logits.grad
    dx_ref = dl @ wr.detach().float()
    dw_ref = dl.t() @ x.detach().float()
    assert (x.grad.float() - dx_ref).abs().max().item() < 2e-2 * max(1.0, dx_ref.abs().max().item())
    assert (wr.grad.float() - dw_ref).abs().max().item() < 2e-2 * max(1.0, dw_ref.abs().max().item())


@pytest.mark.parametrize("tied", [True, False])
def test_chunked_head_cross_entropy_native(tied):
    """LM head + cross entropy over vocabulary chunks on the kernels (GEMM into a [T, chunk] block, row statistics,
    in-place gradient, dX / dW GEMMs accumulating in fp32) against the materialised-logits loss in fp32: values and
    gradients; padding columns, ignored and off-shard targets, a weight with a main_grad buffer."""
    from ironcore_b200.ops import functional as OF
    from ironcore_b200.ops import native

    torch.manual_seed(12)
    t, d, v_local, valid, start, chunk = 300, 256, 1536, 1500, 3072, 512
    targets = torch.randint(start - 200, start + valid + 200, (t,), device="cuda")
    targets[7] = -1
    shape = (v_local, d) if tied else (d, v_local)
    x = torch.randn(t, d, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(*shape, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = None if tied else (torch.randn(v_local, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    bf = b.detach().float().requires_grad_(True) if b is not None else None
    logits = xf @ (wf.t() if tied else wf)
    if bf is not None:
        logits = logits + bf
    ref = OF.cross_entropy(logits, targets, vocab_start=start, vocab_valid=valid)
    got = OF.chunked_head_cross_entropy(x, w, targets, tied=tied, bias=b, vocab_start=start, vocab_valid=valid,
                                        chunk=chunk)
    assert type(got.grad_fn).__name__.startswith("_ChunkedHeadCE")
    assert (got - ref).abs().max().item() < 3e-2
    gw = torch.rand(t, device="cuda")
    (ref * gw).sum().backward()
    (got * gw).sum().backward()
    torch.cuda.synchronize()
    native.check_status()
    for name, a, r in (("dx", x.grad, xf.grad), ("dw", w.grad, wf.grad)) + ((("db", b.grad, bf.grad),) if b is not None else ()):
        scale = r.abs().max().item()
        assert (a.float() - r).abs().max().item() < 2e-2 * max(scale, 1.0), (name, scale)
    # accumulation into the optimizer's fp32 gradient buffer
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.ones(*shape, device="cuda")
    got2 = OF.chunked_head_cross_entropy(x.detach(), w2, targets, tied=tied, bias=None if b is None else b.detach(),
                                         vocab_start=start, vocab_valid=valid, chunk=chunk)
    (got2 * gw).sum().backward()
    torch.cuda.synchronize()
    assert w2.grad is None and w2.grad_ready
    assert (w2.main_grad - 1.0 - wf.grad).abs().max().item() < 2e-2 * max(wf.grad.abs().max().item(), 1.0)
    # without gradients nothing of size [t, v_local] is allocated
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    with torch.no_grad():
        OF.chunked_head_cross_entropy(x, w, targets, tied=tied, bias=b, vocab_start=start, vocab_valid=valid, chunk=chunk)
    assert torch.cuda.max_memory_allocated() - before < t * v_local * 2
