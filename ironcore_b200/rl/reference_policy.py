"""A frozen copy of the policy: the reference model of the KL term (GRPO) and of the log-ratio (DPO)."""

from __future__ import annotations

import torch


def frozen_copy(model, config, loss_fn, device):
    """A second ``LanguageModel`` of the same layout holding the weights ``model`` has now, without gradients
    and in eval mode. It is built, not deep-copied: modules hold process-group handles. The random-number
    state is restored afterwards, so building the copy does not change what the run draws next."""
    from ..models.language_model import LanguageModel

    rng_cpu = torch.get_rng_state()
    rng_dev = torch.cuda.get_rng_state() if device.type == "cuda" else None
    ref = LanguageModel(config, loss_fn, device=device)
    torch.set_rng_state(rng_cpu)
    if rng_dev is not None:
        torch.cuda.set_rng_state(rng_dev)
    with torch.no_grad():
        for dst, src in zip(ref.parameters(), model.parameters()):
            dst.copy_(src)
        for dst, src in zip(ref.buffers(), model.buffers()):
            dst.copy_(src)
    for p in ref.parameters():
        p.requires_grad_(False)
    ref.eval()
    return ref
