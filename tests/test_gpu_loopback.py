"""Fused compute+collective kernels on ONE GPU: a one-rank group runs the whole code path of the fused
reduce-scatter + norm + gather producer (the peer tables point at the GPU's own buffers), and a
"two-rank" call whose second rank does not exist makes the bounded waits run out: the kernels must
return by themselves with a status code, and the device must stay usable."""


import pytest
import torch

from helpers import spawn_gpu_ranks

pytestmark = pytest.mark.gpu


def _rms(h, gamma, eps):
    hf = h.float()
    return hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()


def check_rs_norm_gather_one_rank(rank, world):
    import torch.distributed as dist

    from ironcore_b200.parallel.fused_comm import FusedTP

    torch.manual_seed(5)
    for tokens, d, k, n in ((512, 512, 384, 768), (256, 4096, 256, 512), (384, 2048, 128, 256)):
        ws = FusedTP(tokens, d, dist.group.WORLD, num_slots=2)
        for it in range(3):     # cumulative counters and receive-buffer parity over several calls
            a = torch.randn(tokens, k, device="cuda").bfloat16()
            b = (torch.randn(k, d, device="cuda") / k ** 0.5).bfloat16()
            res = torch.randn(tokens, d, device="cuda").bfloat16()
            gamma = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
            slot = ws.slots[it % 2]
            slot.buf.fill_(float("nan"))
            h, rstd = ws.gemm_rs(a, b, b_major=1, residual=res, norm=(gamma, 1e-5, 0.0, slot))
            ref_h = (a.float() @ b.float() + res.float())
            assert (h.float() - ref_h).abs().max().item() < 0.06
            ref_n = _rms(h, gamma, 1e-5)
            got_n = slot.buf.float()
            assert torch.isfinite(got_n).all()
            assert (got_n - ref_n).abs().max().item() < 0.04 * max(1.0, ref_n.abs().max().item())
            ref_rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5)
            assert torch.allclose(rstd, ref_rstd, rtol=1e-4, atol=1e-6)
            # the consumer waits on the slot's counters only (nothing is pushed) and multiplies
            w = (torch.randn(d, n, device="cuda") / d ** 0.5).bfloat16()
            y = ws.ag_gemm(slot.local, w, a_major=0, b_major=1, n=n, slot=slot, pushed=True)
            assert (y.float() - slot.buf.float() @ w.float()).abs().max().item() < 0.06


def check_rs_norm_autograd_one_rank(rank, world):
    """(h, normed) of the fused op and its gradients against the unfused composition."""
    import torch.distributed as dist

    from ironcore_b200.ops import functional as OF
    from ironcore_b200.parallel.fused_comm import FusedTP

    torch.manual_seed(9)
    tokens, d, k, n = 256, 512, 256, 384
    ws = FusedTP(tokens, d, dist.group.WORLD, num_slots=1)
    slot = ws.slots[0]
    mk = lambda *s, sc=1.0: (torch.randn(*s, device="cuda") * sc).bfloat16().requires_grad_(True)
    x, w, res, gamma, w2 = mk(tokens, k), mk(k, d, sc=k ** -0.5), mk(tokens, d), mk(d, sc=0.2), mk(d, n, sc=d ** -0.5)
    h, normed = ws.linear_reduce_scatter_norm(x, w, None, res, gamma, 1e-5, 1.0, slot)
    y = ws.allgather_linear(normed, w2, None, slot, True)
    loss = (y.float().pow(2).mean() + h.float().mean())
    loss.backward()
    got = [t.grad.float().clone() for t in (x, w, res, gamma, w2)]
    for t in (x, w, res, gamma, w2):
        t.grad = None
    h2 = OF.linear(x, w, None, res)
    n2, _ = OF.norm(h2, gamma, None, 1e-5, True, w_offset=1.0)
    y2 = OF.linear(n2, w2, None)
    (y2.float().pow(2).mean() + h2.float().mean()).backward()
    want = [t.grad.float() for t in (x, w, res, gamma, w2)]
    assert (y.float() - y2.float()).abs().max().item() < 0.05
    for name, a, b in zip(("x", "w", "res", "gamma", "w2"), got, want):
        scale = b.abs().max().item() + 1e-6
        assert (a - b).abs().max().item() < 0.05 * scale, (name, (a - b).abs().max().item(), scale)


def check_row_norm_column_one_rank(rank, world):
    """The whole fused boundary (forward pair and mirrored backward pair of kernels) against the unfused ops:
    outputs and all six gradients, with the residual stream also feeding the loss directly."""
    import torch.distributed as dist

    from ironcore_b200.ops import functional as OF
    from ironcore_b200.parallel.fused_comm import FusedTP

    torch.manual_seed(13)
    for tokens, d, k, n in ((256, 512, 256, 384), (256, 4096, 128, 256)):
        ws = FusedTP(tokens, d, dist.group.WORLD, num_slots=1)
        slot = ws.slots[0]
        mk = lambda *s, sc=1.0: (torch.randn(*s, device="cuda") * sc).bfloat16().requires_grad_(True)
        x, w, res, w2 = mk(tokens, k), mk(k, d, sc=k ** -0.5), mk(tokens, d), mk(d, n, sc=d ** -0.5)
        gamma = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_(True)
        probe = torch.randn(tokens, d, device="cuda").bfloat16()
        for step in range(2):      # twice: cumulative counters, receive-buffer and scratch parity
            for t in (x, w, res, gamma, w2):
                t.grad = None
            h, y = ws.row_norm_column(x, w, None, res, gamma, 1e-5, 0.0, w2, None, slot)
            (y.float().pow(2).mean() + (h.float() * probe.float()).mean()).backward()
            got = [t.grad.float().clone() for t in (x, w, res, gamma, w2)]
            for t in (x, w, res, gamma, w2):
                t.grad = None
            h2 = OF.linear(x, w, None, res)
            n2, _ = OF.norm(h2, gamma, None, 1e-5, True)
            y2 = OF.linear(n2, w2, None)
            (y2.float().pow(2).mean() + (h2.float() * probe.float()).mean()).backward()
            want = [t.grad.float() for t in (x, w, res, gamma, w2)]
            assert (y.float() - y2.float()).abs().max().item() < 0.05
            assert (h.float() - h2.float()).abs().max().item() < 0.05
            for name, a, b in zip(("x", "w", "res", "gamma", "w2"), got, want):
                scale = b.abs().max().item() + 1e-6
                assert (a - b).abs().max().item() < 0.05 * scale, (step, name, (a - b).abs().max().item(), scale)


def check_withheld_peer_flag_times_out(rank, world):
    """A gather over "two ranks" of which only this one exists: the arrival counters of the other rank's
    row blocks never move. With a limit of a few milliseconds the kernel gives up, reports
    kTimeoutPeerFlag and returns; later waits return at once; the device keeps working."""
    import time

    from ironcore_b200.ops import kernels, native
    from ironcore_b200.ops.native import call, ptr, stream_ptr
    from ironcore_b200.parallel import fused_comm  # noqa: F401  (registers the entry points)

    dev = torch.device("cuda")
    rows, d, n, fake_world = 256, 512, 256, 2
    native.set_wait_limit_us(3000)
    try:
        gathered = torch.zeros(fake_world * rows, d, device=dev, dtype=torch.bfloat16)
        gathered[:rows].normal_()
        ready = torch.zeros(fake_world * rows // 128, device=dev, dtype=torch.int32)
        peers = torch.tensor([gathered.data_ptr()] * fake_world, device=dev, dtype=torch.int64)
        peer_ready = torch.tensor([ready.data_ptr()] * fake_world, device=dev, dtype=torch.int64)
        epoch = torch.zeros(1, device=dev, dtype=torch.int32)
        w = torch.randn(d, n, device=dev).bfloat16()
        out = torch.empty(fake_world * rows, n, device=dev, dtype=torch.bfloat16)
        status = native.status_tensor(dev)

        def launch():
            call("icb_ag_gemm", ptr(gathered), ptr(peers), ptr(peer_ready), None, ptr(ready), 0, fake_world, rows, d,
                 ptr(epoch), ptr(w), ptr(out), None, None, n, w.stride(0), out.stride(0), 0, 0, 1, 0, 0, ptr(status),
                 stream_ptr(), None, 0)

        torch.cuda.synchronize()
        t0 = time.perf_counter()
        launch()
        torch.cuda.synchronize()
        first = time.perf_counter() - t0
        code, limit, detail, _ = status.tolist()
        assert code == 5 and limit == 3000, status.tolist()          # kTimeoutPeerFlag
        assert detail >= rows // 128                                  # a row block of the absent rank
        assert first < 1.0, first                                     # one limit, not one per tile
        # the rows that were there are still multiplied correctly
        assert (out[:rows].float() - gathered[:rows].float() @ w.float()).abs().max().item() < 0.3
        # fail fast: with the status word set, the next launch does not wait at all
        t0 = time.perf_counter()
        launch()
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        with pytest.raises(RuntimeError, match="peer flag"):
            native.check_status()
        native.check_status()                                         # cleared by the raise; limit kept
        assert status.tolist()[1] == 3000

        # same for the reduce phase of GEMM -> reduce-scatter: the other rank's partial tiles never arrive
        k = 128
        a = torch.randn(fake_world * rows, k, device=dev).bfloat16()
        b = torch.randn(k, d, device=dev).bfloat16()
        recv = torch.zeros(fake_world, rows, d, device=dev, dtype=torch.bfloat16)
        sink = torch.zeros_like(recv)
        n_flags = (rows // 128) * ((d + 255) // 256)
        flags, sink_flags = (torch.zeros(n_flags, device=dev, dtype=torch.int32) for _ in range(2))
        peer_recv = torch.tensor([recv.data_ptr(), sink.data_ptr()], device=dev, dtype=torch.int64)
        peer_flags = torch.tensor([flags.data_ptr(), sink_flags.data_ptr()], device=dev, dtype=torch.int64)
        out2 = torch.empty(rows, d, device=dev, dtype=torch.bfloat16)
        t0 = time.perf_counter()
        call("icb_gemm_rs", ptr(a), ptr(b), ptr(out2), None, None, fake_world * rows, d, k, a.stride(0), b.stride(0),
             out2.stride(0), 0, 1, 0, ptr(peer_recv), ptr(peer_flags), ptr(recv), ptr(flags), 0, fake_world, ptr(epoch),
             ptr(status), stream_ptr(), None)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0
        assert status.tolist()[0] == 5
        native.clear_status()
        # the context is healthy: an ordinary GEMM gives the right answer
        x = torch.randn(256, 256, device=dev).bfloat16()
        y = kernels.mm_nn(x, x)
        assert (y.float() - x.float() @ x.float()).abs().max().item() < 1.0
    finally:
        native.set_wait_limit_us(0)
        native.clear_status()


def test_rs_norm_gather_one_rank():
    spawn_gpu_ranks("test_gpu_loopback", "check_rs_norm_gather_one_rank", world=1)


def test_rs_norm_autograd_one_rank():
    spawn_gpu_ranks("test_gpu_loopback", "check_rs_norm_autograd_one_rank", world=1)


def test_withheld_peer_flag_times_out():
    spawn_gpu_ranks("test_gpu_loopback", "check_withheld_peer_flag_times_out", world=1)


def test_row_norm_column_one_rank():
    spawn_gpu_ranks("test_gpu_loopback", "check_row_norm_column_one_rank", world=1)
