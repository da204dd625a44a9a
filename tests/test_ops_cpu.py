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
