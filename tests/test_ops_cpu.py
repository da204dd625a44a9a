"""Host-side definitions that the CUDA kernels are tested against."""

import torch


def test_attention_dropout_mask_definition():
    """The host statement of the flash kernels' dropout mask: right keep rate, no structure along rows, columns
    or heads, and a different mask for a different seed."""
    from ironcore_b200.ops.attention import dropout_keep_mask, dropout_threshold

    assert dropout_threshold(0.0) == 0 and dropout_threshold(0.1) == 26 and dropout_threshold(1.0) == 255
    keep = dropout_keep_mask(12345, 2, 3, 200, 0.1).float()
    assert keep.shape == (2, 3, 200, 200)
    assert abs(keep.mean().item() - (1 - 26 / 256)) < 5e-3
    assert (keep.mean(dim=-1) - keep.mean()).abs().max().item() < 0.12       # per query row
    assert (keep.mean(dim=-2) - keep.mean()).abs().max().item() < 0.12       # per key column
    assert not torch.equal(keep[0, 0], keep[0, 1]) and not torch.equal(keep[0], keep[1])
    other = dropout_keep_mask(12346, 2, 3, 200, 0.1).float()
    agree = (other == keep).float().mean().item()
    assert abs(agree - ((1 - 26 / 256) ** 2 + (26 / 256) ** 2)) < 0.01       # independent masks


def _full_head_ce(x, weight, bias, targets, tied, vocab_start, vocab_valid):
    from ironcore_b200.ops import functional as OF

    logits = x @ (weight.t() if tied else weight)
    if bias is not None:
        logits = logits + bias
    return OF.cross_entropy(logits, targets, vocab_start=vocab_start, vocab_valid=vocab_valid)


def test_chunked_head_cross_entropy_matches_materialised():
    """LM head + cross entropy over vocabulary chunks (the logits never exist as a whole) against the same loss
    on materialised logits: values and the gradients of x, the head weight and its bias; tied and untied layouts,
    padding columns, ignored targets, a vocabulary shard that does not start at 0."""
    from ironcore_b200.ops import functional as OF

    torch.manual_seed(3)
    t, d, v_local, valid, start = 37, 48, 640, 600, 1280
    targets = torch.randint(start - 100, start + valid + 100, (t,))      # some targets live on other shards
    targets[5] = -1
    for tied in (True, False):
        shape = (v_local, d) if tied else (d, v_local)
        for with_bias in (False, True):
            leaves = []
            for _ in range(2):
                torch.manual_seed(4)
                x = torch.randn(t, d, dtype=torch.float64, requires_grad=True)
                w = (torch.randn(*shape, dtype=torch.float64) * 0.2).requires_grad_(True)
                b = torch.randn(v_local, dtype=torch.float64, requires_grad=True) if with_bias else None
                leaves.append((x, w, b))
            (x1, w1, b1), (x2, w2, b2) = leaves
            ref = _full_head_ce(x1, w1, b1, targets, tied, start, valid)
            got = OF.chunked_head_cross_entropy(x2, w2, targets, tied=tied, bias=b2, vocab_start=start,
                                                vocab_valid=valid, chunk=256)
            assert torch.allclose(got.double(), ref.double(), atol=1e-5, rtol=1e-5)
            weights = torch.randn(t, dtype=torch.float64)
            (ref.double() * weights).sum().backward()
            (got.double() * weights).sum().backward()
            assert torch.allclose(x2.grad, x1.grad, atol=1e-5, rtol=1e-4)
            assert torch.allclose(w2.grad, w1.grad, atol=1e-5, rtol=1e-4)
            if with_bias:
                assert torch.allclose(b2.grad, b1.grad, atol=1e-5, rtol=1e-4)


def test_accumulate_split_policy():
    """Split of K for in-place fp32 accumulation: only where whole-K tiles fill 148 SMs badly (8-way tensor-parallel
    weight-gradient shards), never for the unsharded layer shapes, and never below 8 k-blocks per work item."""
    from ironcore_b200.ops import kernels

    old = kernels._NUM_SMS
    kernels._NUM_SMS = 148
    try:
        assert kernels._accumulate_split(4096, 1536, 4096) > 1        # qkv shard, 8 ranks
        assert kernels._accumulate_split(512, 4096, 4096) > 1         # attention output shard, 8 ranks
        assert kernels._accumulate_split(1376, 4096, 4096) > 1        # down projection shard, 8 ranks
        for shape in [(4096, 12288, 4096), (4096, 4096, 4096), (11008, 4096, 4096), (4096, 22016, 4096),
                      (4096, 3072, 4096), (4096, 5504, 4096)]:
            assert kernels._accumulate_split(*shape) == 1, shape
        assert kernels._accumulate_split(512, 4096, 512) == 1         # 8 k-blocks: nothing to split
    finally:
        kernels._NUM_SMS = old


def test_op_oracles_agree_with_torch_and_with_each_other():
    """The plain restatements in ``ops/reference.py`` are the oracles of the GPU numerics tests: check them
    against PyTorch's own operators (and the two rotary layouts against each other) in fp64-free fp32."""
    import math

    import torch.nn.functional as F

    from ironcore_b200.ops import functional as OF
    from ironcore_b200.ops import reference as R

    torch.manual_seed(0)
    x = torch.randn(5, 7, 48)
    w, b = torch.randn(48), torch.randn(48)
    assert torch.allclose(R.rms_norm_reference(x, w, 1e-6), torch.nn.functional.rms_norm(x, (48,), w, 1e-6), atol=1e-5)
    assert torch.allclose(R.rms_norm_reference(x, w, 1e-6, w_offset=1.0),
                          torch.nn.functional.rms_norm(x, (48,), w + 1.0, 1e-6), atol=1e-5)
    assert torch.allclose(R.layer_norm_reference(x, w, b, 1e-5), F.layer_norm(x, (48,), w, b, 1e-5), atol=1e-5)
    f, g = x.chunk(2, -1)
    assert torch.allclose(R.glu_reference(x, "swiglu"), F.silu(f) * g)
    assert torch.allclose(R.glu_reference(x, "glu"), F.glu(x, dim=-1))
    assert torch.allclose(R.glu_reference(x, "geglu"), F.gelu(f, approximate="tanh") * g)

    # attention against scaled_dot_product_attention, causal and with grouped keys / values
    q, k, v = torch.randn(2, 9, 4, 16), torch.randn(2, 9, 2, 16), torch.randn(2, 9, 2, 16)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(2, 1),
                                          v.transpose(1, 2).repeat_interleave(2, 1), is_causal=True).transpose(1, 2)
    assert torch.allclose(R.attention_reference(q, k, v, causal=True), want, atol=1e-5)

    # rotary: a rotation (norm preserving, invertible); dot products depend on the position difference only;
    # the interleaved and the half-split layouts are the same map up to the permutation of the head dimension
    pos = torch.arange(9).expand(2, 9)
    r = R.rope_reference(q, pos, 10000.0)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    assert torch.allclose(R.rope_reference(r, pos, 10000.0, inverse=True), q, atol=1e-5)
    q1 = q[:, :1].expand(2, 9, 4, 16).contiguous()          # the same vector at every position
    rq, rk = R.rope_reference(q1, pos, 10000.0), R.rope_reference(q1, pos + 3, 10000.0)
    dots = (rq * rk).sum(-1)                                  # offset 3 everywhere -> the same value everywhere
    assert torch.allclose(dots, dots[:, :1].expand_as(dots), atol=1e-4)
    perm = torch.cat([torch.arange(0, 16, 2), torch.arange(1, 16, 2)])
    assert torch.allclose(R.rope_reference(q, pos, 10000.0)[..., perm],
                          R.rope_reference(q[..., perm], pos, 10000.0, interleaved=False), atol=1e-5)

    # vocabulary-sharded cross entropy against F.cross_entropy, with padding columns and ignored targets
    logits = torch.randn(12, 40)
    tgt = torch.randint(0, 37, (12,))
    tgt[3] = -1
    got = OF.cross_entropy(logits, tgt, vocab_start=0, vocab_valid=37)
    want = F.cross_entropy(logits[:, :37], tgt.clamp_min(0), reduction="none")
    keep = tgt >= 0
    assert torch.allclose(got[keep], want[keep], atol=1e-5) and float(got[3]) == 0.0
    # embedding with a position table
    table, ptab = torch.randn(30, 8), torch.randn(16, 8)
    ids = torch.randint(0, 30, (2, 5))
    pid = torch.arange(5).expand(2, 5)
    assert torch.allclose(OF.embedding(ids, table, pos_table=ptab, pos_ids=pid).view(2, 5, 8), table[ids] + ptab[pid])
    assert math.isfinite(float(got.sum()))


def test_fallbacks_are_reported_once_and_only_for_native_candidates(monkeypatch):
    """``note_fallback`` warns once per (op, reason) and stays silent for tensors that never had a native path."""
    import warnings

    from ironcore_b200.ops import functional as OF

    monkeypatch.setattr(OF, "_FALLBACKS_SEEN", set())
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        OF.norm(torch.randn(4, 12), torch.ones(12), None, 1e-5, True)          # CPU fp32: nothing to report
        OF.note_fallback("norm", "row length 12 is not a multiple of 8 up to 8192", torch.randn(2))
        assert not seen
        OF.note_fallback("norm", "row length 12 is not a multiple of 8 up to 8192")
        OF.note_fallback("norm", "row length 12 is not a multiple of 8 up to 8192")
        assert len(seen) == 1 and "native sm_100a kernel" in str(seen[0].message)
