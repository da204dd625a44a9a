"""tcgen05 GEMM against an fp32 PyTorch reference: every operand-major combination,
ragged shapes, epilogue options and the grouped (mixture-of-experts) forms."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_major, b_major):
    A = a.float() if a_major == 0 else a.float().t()
    B = b.float().t() if b_major == 0 else b.float()
    return A @ B


def _mk(rows, cols, dtype=torch.bfloat16, scale=1.0):
    return (torch.randn(rows, cols, device="cuda") * scale).to(dtype)


def _check(out, ref, k, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    bound = tol * (k ** 0.5)
    assert err <= bound, f"max abs err {err} > {bound}"


@pytest.mark.parametrize("a_major,b_major", [(0, 1), (0, 0), (1, 1), (1, 0)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (384, 1376, 520), (200, 264, 72), (4096, 1536, 1024)])
def test_gemm_majors(a_major, b_major, m, n, k):
    from ironcore_b200.ops import kernels, native

    torch.manual_seed(0)
    a = _mk(m, k) if a_major == 0 else _mk(k, m)
    b = _mk(n, k) if b_major == 0 else _mk(k, n)
    out = kernels.gemm(a, b, a_major=a_major, b_major=b_major, m=m, n=n, k=k)
    torch.cuda.synchronize()
    native.check_status()
    _check(out, _ref(a, b, a_major, b_major), k)


def test_gemm_epilogue_bias_residual_fp32():
    from ironcore_b200.ops import kernels, native

    torch.manual_seed(1)
    m, n, k = 300, 520, 256
    x, w = _mk(m, k), _mk(k, n)
    bias = _mk(1, n).reshape(n)
    res = _mk(m, n)
    out = kernels.mm_nn(x, w, bias=bias, residual=res)
    ref = x.float() @ w.float() + bias.float() + res.float()
    _check(out, ref, k)
    # fp32 output with in-place accumulation (C += A B)
    acc = torch.randn(m, n, device="cuda")
    ref2 = acc + x.float() @ w.float()
    out2 = kernels.mm_nn(x, w, out=acc, residual=acc, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.check_status()
    assert out2.data_ptr() == acc.data_ptr()
    _check(out2, ref2, k, tol=1e-2)


@pytest.mark.parametrize("m,n,k", [(64, 2048, 1536), (64, 1536, 8960), (8, 17920, 1536), (130, 520, 1000)])
def test_gemm_split_k_small_m(m, n, k):
    """Decode-shaped products (a few token rows against a wide weight matrix) take the split-K path: the K
    ranges of one output tile are computed by different CTAs and accumulated with TMA reduce-add."""
    from ironcore_b200.ops import kernels, native

    torch.manual_seed(2)
    assert kernels._split_k_for(m, n, k) > 1
    x, w = _mk(m, k), _mk(k, n, scale=k ** -0.5)
    bias = _mk(1, n).reshape(n)
    res = _mk(m, n)
    ref = x.float() @ w.float()
    _check(kernels.mm_nn(x, w), ref, k)
    _check(kernels.mm_nn(x, w, bias=bias, residual=res), ref + bias.float() + res.float(), k)
    wt = w.t().contiguous()                               # [n, k]: the dgrad / tied-head orientation
    _check(kernels.mm_nt(x, wt), ref, k)
    # run to run the accumulation order of the K ranges may differ: results agree to fp32 rounding
    a, b = kernels.mm_nn(x, w), kernels.mm_nn(x, w)
    assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item()
    torch.cuda.synchronize()
    native.check_status()


def test_gemm_fp16():
    from ironcore_b200.ops import kernels

    torch.manual_seed(2)
    m, n, k = 256, 256, 128
    x, w = _mk(m, k, torch.float16), _mk(k, n, torch.float16)
    out = kernels.mm_nn(x, w)
    _check(out, x.float() @ w.float(), k, tol=5e-3)


def test_gemm_backward_helpers():
    from ironcore_b200.ops import kernels

    torch.manual_seed(3)
    m, k, n = 512, 264, 392
    x, w, dy = _mk(m, k), _mk(k, n), _mk(m, n)
    _check(kernels.mm_nt(dy, w), dy.float() @ w.float().t(), n)
    _check(kernels.mm_tn(x, dy), x.float().t() @ dy.float(), m)


def test_gemm_grouped_by_m_tile():
    from ironcore_b200.ops import kernels

    torch.manual_seed(4)
    g, k, n = 3, 128, 320
    rows = [256, 128, 384]
    table = torch.tensor([0, 0, 1, 2, 2, 2], dtype=torch.int32, device="cuda")
    m = sum(rows)
    x = _mk(m, k)
    w = (torch.randn(g, k, n, device="cuda")).to(torch.bfloat16)
    out = kernels.gemm(x, w, a_major=0, b_major=1, m=m, n=n, k=k, group_mode=1, num_groups=g,
                       group_table=table, b_group_stride=k * n)
    ref = torch.cat([x[:256].float() @ w[0].float(), x[256:384].float() @ w[1].float(), x[384:].float() @ w[2].float()])
    _check(out, ref, k)


def test_gemm_grouped_by_k_range():
    from ironcore_b200.ops import kernels

    torch.manual_seed(5)
    g, kin, n = 3, 200, 264
    offs = torch.tensor([0, 128, 128, 448], dtype=torch.int32, device="cuda")  # middle group is empty
    x = _mk(448, kin)
    dy = _mk(448, n)
    out = kernels.gemm(x, dy, a_major=1, b_major=1, m=kin, n=n, k=448, group_mode=2, num_groups=g, group_table=offs)
    refs = [x[0:128].float().t() @ dy[0:128].float(), torch.zeros(kin, n, device="cuda"),
            x[128:448].float().t() @ dy[128:448].float()]
    for i in range(g):
        _check(out[i], refs[i], 320)


@pytest.mark.parametrize("a_major,b_major", [(0, 1), (0, 0), (1, 1), (1, 0)])
def test_gemm_2sm_matches_reference(a_major, b_major):
    """256 x 256 tiles on CTA pairs (tcgen05.mma.cta_group::2) against fp32 matmul, ragged edges included."""
    from ironcore_b200.ops import native
    from ironcore_b200.ops.native import call, dtype_code, ptr, stream_ptr
    from ironcore_b200.ops import kernels  # noqa: F401  (registers icb_gemm_2sm)

    torch.manual_seed(3)
    native.set_wait_limit_us(200000)     # a protocol mistake in the pair ends after 0.2 s per wait, not 2 s
    for (m, n, k) in [(256, 256, 64), (512, 768, 256), (384, 320, 192), (4096, 1536, 1024)]:
        a = torch.randn((m, k) if a_major == 0 else (k, m), device="cuda").bfloat16()
        b = torch.randn((n, k) if b_major == 0 else (k, n), device="cuda").bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        call("icb_gemm_2sm", ptr(a), ptr(b), ptr(out), None, None, m, n, k, a.stride(0), b.stride(0), out.stride(0), 0,
             a_major, b_major, dtype_code(torch.bfloat16), 0, ptr(native.status_tensor(a.device)), stream_ptr())
        torch.cuda.synchronize()
        native.check_status()
        af = a.float() if a_major == 0 else a.float().t()
        bf = b.float().t() if b_major == 0 else b.float()
        ref = af @ bf
        err = (out.float() - ref).abs().max().item()
        assert err <= 2e-2 * (k ** 0.5) + 2.0 ** -7 * ref.abs().max().item(), (m, n, k, err)
    native.set_wait_limit_us(0)


def test_gemm_2sm_epilogue_and_policy():
    """Bias, residual and in-place fp32 accumulation on the CTA-pair kernel, and the automatic choice:
    large plain problems take the pair kernel, small and grouped ones the single-CTA kernel; both agree."""
    from ironcore_b200.ops import kernels, native

    torch.manual_seed(8)
    m, n, k = 1024, 1280, 512
    x, w = _mk(m, k), _mk(k, n)
    bias, res = _mk(1, n).reshape(n), _mk(m, n)
    ref = x.float() @ w.float() + bias.float() + res.float()
    assert kernels._two_sm_wins(m, n, k) and not kernels._two_sm_wins(256, 256, 64)
    a = kernels.mm_nn(x, w, bias=bias, residual=res, two_sm=True)
    b = kernels.mm_nn(x, w, bias=bias, residual=res, two_sm=False)
    c = kernels.mm_nn(x, w, bias=bias, residual=res)            # policy: auto
    _check(a, ref, k)
    _check(b, ref, k)
    assert torch.equal(a, c)
    acc = torch.randn(k, n, device="cuda")
    dy = _mk(m, n)
    ref2 = acc + x.float().t() @ dy.float()
    out = kernels.mm_tn(x, dy, out=acc, residual=acc, out_dtype=torch.float32, two_sm=True)
    torch.cuda.synchronize()
    native.check_status()
    assert out.data_ptr() == acc.data_ptr()
    _check(out, ref2, m, tol=1e-2)


def test_gemm_accumulate_in_place_splits_k():
    """C += A^T B with an fp32 C (the weight-gradient form): shapes whose whole-K tiles fill the machine badly
    split the K range over several CTAs that add into C with TMA reduce-adds; same result as the unsplit kernels."""
    from ironcore_b200.ops import kernels, native

    torch.manual_seed(9)
    m, n, k = 512, 4096, 4096          # an 8-way shard of the attention output projection's gradient
    assert kernels._accumulate_split(m, n, k) > 1 and kernels._accumulate_split(4096, 4096, 4096) == 1
    x, dy = _mk(k, m), _mk(k, n)
    start = torch.randn(m, n, device="cuda")
    ref = start + x.float().t() @ dy.float()
    acc = start.clone()
    out = kernels.mm_tn(x, dy, out=acc, residual=acc, out_dtype=torch.float32)          # policy: split
    pair = start.clone()
    kernels.mm_tn(x, dy, out=pair, residual=pair, out_dtype=torch.float32, two_sm=True)  # forced: CTA pairs
    torch.cuda.synchronize()
    native.check_status()
    assert out.data_ptr() == acc.data_ptr()
    _check(acc, ref, k, tol=1e-2)
    assert (acc - pair).abs().max().item() <= 1e-3 * ref.abs().max().item()
