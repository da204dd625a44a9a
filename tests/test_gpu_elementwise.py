"""Norm / RoPE / activation / embedding / cross-entropy / Adam kernels against fp32
PyTorch restatements of the same math."""

import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _close(a, b, atol, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    assert bool((err <= lim).all()), f"max err {err.max().item()} (ref max {b.abs().max().item()})"


@pytest.mark.parametrize("rms", [True, False])
@pytest.mark.parametrize("m,d", [(64, 768), (300, 4096), (17, 1536), (8, 8192)])
def test_norm_fwd_bwd(rms, m, d):
    from ironcore_b200.ops import kernels

    torch.manual_seed(0)
    x = torch.randn(m, d, device="cuda").to(BF)
    res = torch.randn(m, d, device="cuda").to(BF)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(BF)
    b = None if rms else (0.1 * torch.randn(d, device="cuda")).to(BF)
    dy = torch.randn(m, d, device="cuda").to(BF)
    y, h, mean, rstd = kernels.norm_fwd(x, w, b, 1e-5, rms, residual=res)
    hf = (x.float() + res.float()).to(BF).float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    bf = b.float().requires_grad_(True) if b is not None else None
    if rms:
        ref = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    else:
        ref = F.layer_norm(hf, (d,), wf, bf, 1e-5)
    _close(h, hf.detach(), 1e-6, 1e-6)
    _close(y, ref, 2e-2)
    ref.backward(dy.float())
    dx, dw, db = kernels.norm_bwd(dy, h, w, mean, rstd, rms, has_bias=b is not None)
    _close(dx, hf.grad, 3e-2)
    _close(dw, wf.grad, 2e-2 * math.sqrt(m), 1e-2)
    if b is not None:
        _close(db, bf.grad, 2e-2 * math.sqrt(m), 1e-2)


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_roundtrip_and_reference(interleaved):
    from ironcore_b200.ops import kernels

    torch.manual_seed(1)
    b, s, h, hd = 2, 96, 4, 128
    x = torch.randn(b * s, h, hd, device="cuda").to(BF)
    out = torch.empty_like(x)
    kernels.rope(x, out, nheads=h, head_dim=hd, tokens=b * s, seq_len=s, base=10000.0, interleaved=interleaved)
    pos = torch.arange(s, device="cuda").repeat(b).float()
    inv = 10000.0 ** (-torch.arange(0, hd, 2, device="cuda").float() / hd)
    ang = pos[:, None] * inv[None, :]
    c, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    if interleaved:
        x0, x1 = xf[..., 0::2], xf[..., 1::2]
        ref = torch.stack([x0 * c - x1 * sn, x1 * c + x0 * sn], dim=-1).flatten(-2)
    else:
        x0, x1 = xf[..., : hd // 2], xf[..., hd // 2:]
        ref = torch.cat([x0 * c - x1 * sn, x1 * c + x0 * sn], dim=-1)
    _close(out, ref, 2e-2)
    back = torch.empty_like(x)
    kernels.rope(out, back, nheads=h, head_dim=hd, tokens=b * s, seq_len=s, base=10000.0, interleaved=interleaved,
                 inverse=True)
    _close(back, xf, 3e-2)


@pytest.mark.parametrize("interleaved", [True, False])
def test_partial_rotary_in_place_and_attention(interleaved):
    """Phi-style partial rotary: the first rot_dim elements of every head rotate (frequencies over rot_dim), the
    rest stays; and the attention op keeps such models on the flash kernel."""
    from ironcore_b200.ops import functional as OF
    from ironcore_b200.ops import kernels, reference

    torch.manual_seed(2)
    b, s, h, hd, rot = 2, 64, 4, 64, 32
    x = torch.randn(b * s, h, hd, device="cuda").to(BF)
    ref = x.clone()
    pos = torch.arange(s, device="cuda").repeat(b)
    ref[..., :rot] = reference.rope_reference(x[..., :rot], pos, 10000.0, 1.0, 0, interleaved)
    y = x.clone()
    kernels.rope(y, y, nheads=h, head_dim=hd, tokens=b * s, seq_len=s, base=10000.0, interleaved=interleaved, rot_dim=rot)
    _close(y, ref.float(), 2e-2)
    assert torch.equal(y[..., rot:], x[..., rot:])
    qkv = (0.5 * torch.randn(b * s, 3 * h * hd, device="cuda")).to(BF).requires_grad_(True)
    rope = (10000.0, 1.0, 0, interleaved, None)
    qf = qkv.detach().float().requires_grad_(True)
    # the op rotates its input in place (it owns the projection output), so it is given a copy of the leaf
    out = OF.rope_attention(qkv * 1.0, num_heads=h, num_kv_heads=h, head_dim=hd, seq_len=s, rope=rope, rot_dim=rot)
    want = OF.rope_attention(qf, num_heads=h, num_kv_heads=h, head_dim=hd, seq_len=s, rope=rope, rot_dim=rot, fused=False)
    _close(out, want, 3e-2)
    g = torch.randn_like(out)
    out.backward(g)
    want.backward(g.float())
    _close(qkv.grad, qf.grad, 6e-2)


@pytest.mark.parametrize("name", ["swiglu", "geglu", "geglu_erf", "reglu", "glu"])
def test_glu(name):
    from ironcore_b200.ops import kernels
    from ironcore_b200.ops.reference import glu_reference

    torch.manual_seed(2)
    m, f = 130, 1376
    x = torch.randn(m, 2 * f, device="cuda").to(BF)
    dy = torch.randn(m, f, device="cuda").to(BF)
    y = kernels.glu_fwd(x, name)
    xf = x.float().requires_grad_(True)
    ref = glu_reference(xf, name)
    _close(y, ref, 2e-2)
    ref.backward(dy.float())
    dx = kernels.glu_bwd(dy, x, name)
    _close(dx, xf.grad, 3e-2)
    # a row limit: rows from it on may hold anything (NaN here); they come out as zeros, the others unchanged
    limit = torch.tensor([77], dtype=torch.int32, device="cuda")
    xn = x.clone()
    xn[77:] = float("nan")
    y2 = kernels.glu_fwd(xn, name, limit)
    dx2 = kernels.glu_bwd(dy, xn, name, limit)
    assert torch.equal(y2[:77], y[:77]) and torch.equal(dx2[:77], dx[:77])
    assert not y2[77:].any() and not dx2[77:].any()


@pytest.mark.parametrize("name", ["relu", "gelu", "gelu_tanh", "silu"])
def test_act(name):
    from ironcore_b200.ops import kernels
    from ironcore_b200.ops.reference import act_reference

    torch.manual_seed(3)
    x = torch.randn(64, 3072, device="cuda").to(BF)
    dy = torch.randn(64, 3072, device="cuda").to(BF)
    xf = x.float().requires_grad_(True)
    ref = act_reference(xf, name)
    _close(kernels.act_fwd(x, name), ref, 2e-2)
    ref.backward(dy.float())
    _close(kernels.act_bwd(dy, x, name), xf.grad, 3e-2)


def test_embedding_fwd_bwd():
    from ironcore_b200.ops import kernels

    torch.manual_seed(4)
    v, d, s = 1000, 768, 64
    w = torch.randn(v, d, device="cuda").to(BF)
    pt = torch.randn(s, d, device="cuda").to(BF)
    ids = torch.randint(0, 2 * v, (3, s), device="cuda")
    out = kernels.embedding_fwd(ids, w, vocab_start=500, pos_table=pt, seq_len=s)
    local = ids - 500
    ok = (local >= 0) & (local < v)
    ref = torch.where(ok[..., None], w.float()[local.clamp(0, v - 1)], torch.zeros((), device="cuda"))
    ref = ref + pt.float()[None]
    _close(out, ref, 2e-2)
    dy = torch.randn(3, s, d, device="cuda").to(BF)
    dw = kernels.embedding_bwd(ids, dy, v, row_start=500)
    refdw = torch.zeros(v, d, device="cuda")
    refdw.index_add_(0, local[ok], dy.float()[ok])
    _close(dw, refdw, 1e-3, 1e-3)


@pytest.mark.parametrize("t,v,valid", [(33, 32000, 32000), (7, 50304, 50257), (5, 1000, 1000)])
def test_cross_entropy(t, v, valid):
    from ironcore_b200.ops import kernels

    torch.manual_seed(5)
    logits = (3 * torch.randn(t, v, device="cuda")).to(BF)
    tgt = torch.randint(0, valid, (t,), device="cuda")
    rmax, rsum, rtgt = kernels.ce_stats(logits, tgt, vocab_valid=valid)
    lf = logits.float()[:, :valid].requires_grad_(True)
    ref = F.cross_entropy(lf, tgt, reduction="none")
    lse = rmax + rsum.log()
    _close(lse - rtgt, ref, 2e-3, 1e-3)
    gs = torch.rand(t, device="cuda")
    ref.backward(gs)
    g = kernels.ce_grad_(logits.clone(), tgt, lse, gs, vocab_valid=valid)
    _close(g[:, :valid], lf.grad, 2e-3, 2e-2)
    assert float(g[:, valid:].float().abs().max() if valid < v else 0.0) == 0.0


@pytest.mark.parametrize("skew", [0, 1])
def test_adam_and_norms(skew):
    """skew = 0: aligned buffers (four-element kernel plus a three-element tail); skew = 1: views that start one
    element into their buffers, which only the element-wise kernel can take."""
    from ironcore_b200.ops import kernels

    torch.manual_seed(6)
    n = 100_003
    p = torch.randn(n + skew, device="cuda").to(BF)[skew:]
    g = (0.1 * torch.randn(n + skew, device="cuda")).to(BF)[skew:]
    m = torch.zeros(n + skew, device="cuda")[skew:]
    v = torch.zeros(n + skew, device="cuda")[skew:]
    total = torch.zeros(1, device="cuda")
    kernels.sumsq(g, total)
    assert abs(total.item() - g.float().pow(2).sum().item()) < 1e-3 * total.item()
    norm, coef = kernels.clip_coef(total, 1.0)
    assert abs(norm.item() - g.float().norm().item()) < 1e-3 * norm.item()
    pf, gf = p.float(), g.float() * coef.item()
    mf, vf = torch.zeros_like(pf), torch.zeros_like(pf)
    lr, b1, b2, eps, wd = 3e-4, 0.9, 0.95, 1e-8, 0.1
    for step in (1, 2):
        kernels.adam_step_(p, g, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=step,
                           grad_scale_dev=coef)
        mf = b1 * mf + (1 - b1) * gf
        vf = b2 * vf + (1 - b2) * gf * gf
        ss = lr * math.sqrt(1 - b2 ** step) / (1 - b1 ** step)
        pf = (pf * (1 - lr * wd) - ss * mf / (vf.sqrt() + eps)).to(BF).float()
    _close(m, mf, 1e-6, 1e-4)
    _close(v, vf, 1e-9, 1e-4)
    _close(p, pf, 1e-2, 1e-2)
