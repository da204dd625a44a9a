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
