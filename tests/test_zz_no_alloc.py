"""The allocation-free norm-backward entry point, called through its exported C symbol, must
agree with the regular entry point (which takes a caller-provided scratch buffer).

Why the entry point exists: some callers may not allocate device memory when they need this
kernel (a host that fixes all GPU memory at start-up, code living inside another framework's
pool, a loop where an allocator call is not acceptable), so its scratch is a fixed array inside
the library. The array is shared by every call and keeps the previous call's contents; two
calls in a row with different shapes check that nothing stale leaks into the result.
This file is collected last so that a stop-at-first-failure run has already covered the rest."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, dy, x, w, mean, rstd, rms, has_bias):
    m, d = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty(d, dtype=torch.float32, device=x.device)
    db = torch.empty(d, dtype=torch.float32, device=x.device) if has_bias else None
    fn = lib.icb_norm_bwd_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 9 + [C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    p = lambda t: None if t is None else t.data_ptr()
    rc = fn(p(dy), p(x), p(w), p(mean), p(rstd), None, p(dx), p(dw), p(db), m, d, 0.0, 1 if rms else 0, 0, 1, 0,
            torch.cuda.current_stream().cuda_stream)
    return rc, dx, dw, db


@pytest.mark.parametrize("rms", [True, False])
def test_noalloc_matches_regular_entry_point_twice(rms):
    from ironcore_b200.ops import kernels, native

    lib = native.load(strict=True)
    torch.manual_seed(11)
    for m, d in ((777, 4096), (130, 1536)):   # second call is smaller: stale partial rows must not matter
        x = torch.randn(m, d, device="cuda").bfloat16()
        dy = torch.randn(m, d, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
        b = None if rms else (0.1 * torch.randn(d, device="cuda")).bfloat16()
        _y, _h, mean, rstd = kernels.norm_fwd(x, w, b, 1e-5, rms)
        ref_dx, ref_dw, ref_db = kernels.norm_bwd(dy, x, w, mean, rstd, rms, has_bias=b is not None)
        rc, dx, dw, db = _call_noalloc(lib, dy, x, w, mean, rstd, rms, b is not None)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(dx, ref_dx)
        tol = dict(atol=2e-2 * (m ** 0.5), rtol=1e-2)
        assert torch.allclose(dw, ref_dw, **tol), (dw - ref_dw).abs().max().item()
        if b is not None:
            assert torch.allclose(db, ref_db, **tol)


def test_noalloc_rejects_rows_beyond_the_builtin_scratch():
    from ironcore_b200.ops import native

    lib = native.load(strict=True)
    m, d = 8, 8192
    x = torch.randn(m, d, device="cuda").bfloat16()
    w = torch.ones(d, device="cuda").bfloat16()
    rstd = torch.ones(m, device="cuda")
    rc, _dx, _dw, _db = _call_noalloc(lib, x, x, w, None, rstd, True, False)
    assert rc == -20
