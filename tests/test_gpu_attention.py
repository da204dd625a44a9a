"""Flash attention forward / backward against an fp32 PyTorch restatement."""

import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _ref(qkv, b, s, hq, hkv, hd, causal, cu=None):
    from ironcore_b200.ops.functional import document_mask
    from ironcore_b200.ops.reference import attention_reference

    x = qkv.float().view(b, s, hq + 2 * hkv, hd)
    q, k, v = x[:, :, :hq], x[:, :, hq:hq + hkv], x[:, :, hq + hkv:]
    mask = document_mask(cu, b, s, qkv.device) if cu is not None else None
    return attention_reference(q, k, v, causal=causal, mask=mask)


def _err(a, b):
    return (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("b,s,hq,hkv,hd,causal", [
    (1, 128, 1, 1, 128, True), (2, 256, 4, 4, 128, True), (1, 512, 8, 2, 128, True), (2, 384, 4, 4, 64, True),
    (1, 200, 2, 1, 128, True), (1, 320, 2, 2, 64, False), (1, 1024, 4, 1, 128, True),
])
def test_flash_fwd_bwd(b, s, hq, hkv, hd, causal):
    from ironcore_b200.ops import attention, native

    torch.manual_seed(0)
    t = b * s
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda").to(BF)
    dout = torch.randn(t, hq * hd, device="cuda").to(BF)
    out, lse = attention.flash_fwd(qkv, hq, hkv, hd, s, causal=causal)
    torch.cuda.synchronize()
    native.check_status()
    leaf = qkv.float().requires_grad_(True)
    ref = _ref(leaf, b, s, hq, hkv, hd, causal).reshape(t, hq * hd)
    assert _err(out, ref) < 2e-2, f"fwd err {_err(out, ref)}"
    ref.backward(dout.float())
    dqkv = attention.flash_bwd(dout, qkv, out, lse, hq, hkv, hd, s, causal=causal)
    torch.cuda.synchronize()
    native.check_status()
    g = leaf.grad
    nq = hq * hd
    nk = hkv * hd
    scale = g.abs().max().item()
    for name, lo, hi in (("dq", 0, nq), ("dk", nq, nq + nk), ("dv", nq + nk, nq + 2 * nk)):
        e = _err(dqkv[:, lo:hi], g[:, lo:hi])
        assert e < 3e-2 * max(scale, 1.0), f"{name} err {e} (grad scale {scale})"


def test_flash_document_boundaries():
    from ironcore_b200.ops import attention

    torch.manual_seed(1)
    b, s, hq, hkv, hd = 2, 256, 2, 2, 128
    t = b * s
    cu = torch.tensor([0, 100, 256, 300, 512], dtype=torch.int32, device="cuda")
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda").to(BF)
    out, lse = attention.flash_fwd(qkv, hq, hkv, hd, s, cu_seqlens=cu, max_seqlen=256)
    leaf = qkv.float().requires_grad_(True)
    ref = _ref(leaf, b, s, hq, hkv, hd, True, cu=cu).reshape(t, hq * hd)
    assert _err(out, ref) < 2e-2
    dout = torch.randn(t, hq * hd, device="cuda").to(BF)
    ref.backward(dout.float())
    dqkv = attention.flash_bwd(dout, qkv, out, lse, hq, hkv, hd, s, cu_seqlens=cu, max_seqlen=256)
    assert _err(dqkv, leaf.grad) < 3e-2 * max(leaf.grad.abs().max().item(), 1.0)


def test_rope_attention_autograd_matches_reference():
    from ironcore_b200.ops import functional as OF

    torch.manual_seed(2)
    b, s, hq, hkv, hd = 2, 256, 4, 2, 128
    t = b * s
    base = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda")
    rope = (10000.0, 1.0, 0, True, None)
    x1 = base.to(BF).requires_grad_(True)
    y1 = OF.rope_attention(x1 * 1.0, num_heads=hq, num_kv_heads=hkv, head_dim=hd, seq_len=s, rope=rope)
    x2 = base.to(BF).float().requires_grad_(True)
    y2 = OF.rope_attention(x2, num_heads=hq, num_kv_heads=hkv, head_dim=hd, seq_len=s, rope=rope, fused=False)
    assert _err(y1, y2) < 2e-2
    dy = torch.randn_like(y2)
    y1.backward(dy.to(BF))
    y2.backward(dy)
    assert _err(x1.grad, x2.grad) < 3e-2 * max(x2.grad.abs().max().item(), 1.0)


@pytest.mark.parametrize("b,s,hq,hkv,hd,causal,p", [
    (2, 256, 4, 2, 128, True, 0.1), (1, 200, 2, 2, 64, True, 0.25), (1, 384, 2, 1, 128, False, 0.1),
])
def test_flash_dropout_matches_masked_reference(b, s, hq, hkv, hd, causal, p):
    """Dropout inside the kernels: forward and backward recompute the same hash mask; the oracle applies that
    mask (built on the host from the published definition) to an fp32 softmax."""
    from ironcore_b200.ops import attention, native

    torch.manual_seed(5)
    t = b * s
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda").to(BF)
    dout = torch.randn(t, hq * hd, device="cuda").to(BF)
    seed = torch.tensor([0x1234_5678_9ABC], dtype=torch.int64, device="cuda")
    out, lse = attention.flash_fwd(qkv, hq, hkv, hd, s, causal=causal, dropout_p=p, dropout_seed=seed)
    out_nodrop, lse_nodrop = attention.flash_fwd(qkv, hq, hkv, hd, s, causal=causal)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(lse, lse_nodrop)                      # the row statistics ignore the mask
    assert not torch.equal(out, out_nodrop)

    thr = attention.dropout_threshold(p)
    keep = attention.dropout_keep_mask(int(seed.item()), b, hq, s, p).cuda()
    frac = keep.float().mean().item()
    assert abs(frac - (1 - thr / 256)) < 0.01
    leaf = qkv.float().requires_grad_(True)
    x = leaf.view(b, s, hq + 2 * hkv, hd)
    q, k, v = x[:, :, :hq].transpose(1, 2), x[:, :, hq:hq + hkv].transpose(1, 2), x[:, :, hq + hkv:].transpose(1, 2)
    k, v = k.repeat_interleave(hq // hkv, dim=1), v.repeat_interleave(hq // hkv, dim=1)
    scores = q @ k.transpose(-1, -2) * hd ** -0.5
    if causal:
        scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    probs = torch.softmax(scores, dim=-1) * keep * (256.0 / (256 - thr))
    ref = (probs @ v).transpose(1, 2).reshape(t, hq * hd)
    assert _err(out, ref) < 3e-2, f"fwd err {_err(out, ref)}"
    ref.backward(dout.float())
    dqkv = attention.flash_bwd(dout, qkv, out, lse, hq, hkv, hd, s, causal=causal, dropout_p=p, dropout_seed=seed)
    torch.cuda.synchronize()
    native.check_status()
    g = leaf.grad
    nq, nk = hq * hd, hkv * hd
    scale = g.abs().max().item()
    for name, lo, hi in (("dq", 0, nq), ("dk", nq, nq + nk), ("dv", nq + nk, nq + 2 * nk)):
        e = _err(dqkv[:, lo:hi], g[:, lo:hi])
        assert e < 3e-2 * max(scale, 1.0), f"{name} err {e} (grad scale {scale})"


def test_rope_attention_dropout_uses_flash_and_advances_the_mask():
    """The public op keeps dropout on the flash path in training (no score matrix), draws a new mask per call
    and none in evaluation."""
    from ironcore_b200.ops import functional as OF

    torch.manual_seed(6)
    s, hq, hkv, hd = 256, 4, 2, 128
    qkv = torch.randn(s, (hq + 2 * hkv) * hd, device="cuda").to(BF).requires_grad_(True)
    kw = dict(num_heads=hq, num_kv_heads=hkv, head_dim=hd, seq_len=s)
    base = OF.rope_attention(qkv, dropout_p=0.2, training=False, **kw)
    a = OF.rope_attention(qkv, dropout_p=0.2, training=True, **kw)
    b2 = OF.rope_attention(qkv, dropout_p=0.2, training=True, **kw)
    assert type(a.grad_fn).__name__.startswith("_RopeAttention")
    assert torch.equal(base, OF.rope_attention(qkv, **kw))
    assert not torch.equal(a, b2) and not torch.equal(a, base)
    a.float().square().mean().backward()
    assert torch.isfinite(qkv.grad).all() and qkv.grad.abs().max().item() > 0
