"""Paged KV-cache kernels, the GRPO loss kernel and the rollout engine on the GPU."""

import pytest
import torch

from helpers import tiny_config

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("hq,hkv,hd,bs", [(12, 2, 128, 16), (4, 4, 64, 16), (8, 1, 128, 32)])
def test_paged_decode_matches_reference(hq, hkv, hd, bs):
    from ironcore_b200.rl import ops as RO

    torch.manual_seed(0)
    s, max_blocks, nblocks = 5, 8, 64
    kc = torch.randn(nblocks, bs, hkv, hd, device="cuda").to(BF)
    vc = torch.randn(nblocks, bs, hkv, hd, device="cuda").to(BF)
    perm = torch.randperm(nblocks, device="cuda")[: s * max_blocks].view(s, max_blocks).to(torch.int32)
    lens = torch.tensor([1, 17, bs * 3, bs * 8, 50], dtype=torch.int32, device="cuda").clamp(max=bs * max_blocks)
    q = torch.randn(s, hq * hd, device="cuda").to(BF)
    out = RO.paged_decode(q, kc, vc, perm, lens, hq, hkv, hd)
    ref = RO.paged_decode_reference(q, kc, vc, perm, lens, hq, hkv, hd, hd ** -0.5)
    assert (out.float() - ref.float()).abs().max().item() < 2e-2


def test_kv_append_scatter():
    from ironcore_b200.rl import ops as RO

    torch.manual_seed(1)
    t, hkv, hd, bs, nb = 37, 2, 128, 16, 8
    packed = torch.randn(t, 4 * hkv * hd, device="cuda").to(BF)
    k, v = packed[:, hkv * hd:2 * hkv * hd], packed[:, 2 * hkv * hd:3 * hkv * hd]
    kc = torch.zeros(nb, bs, hkv, hd, device="cuda", dtype=BF)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * bs, device="cuda")[:t]
    slots[3] = -1
    RO.kv_append(k, v, kc, vc, slots)
    ok = slots >= 0
    assert torch.equal(kc.view(-1, hkv * hd)[slots[ok]], k[ok])
    assert torch.equal(vc.view(-1, hkv * hd)[slots[ok]], v[ok])


def test_grpo_loss_kernel_matches_formula():
    from ironcore_b200.rl import ops as RO

    torch.manual_seed(2)
    n = 1000
    lp = torch.randn(n, device="cuda").requires_grad_(True)
    old = lp.detach() + 0.3 * torch.randn(n, device="cuda")
    ref = lp.detach() + 0.2 * torch.randn(n, device="cuda")
    adv = torch.randn(n, device="cuda")
    mask = (torch.rand(n, device="cuda") > 0.2).float()
    loss, ratio, kl = RO.grpo_token_loss(lp, old, ref, adv, mask, 0.2, 0.04)
    lp2 = lp.detach().clone().requires_grad_(True)
    r = torch.exp(lp2 - old)
    pg = -torch.minimum(r * adv, r.clamp(0.8, 1.2) * adv)
    d = ref - lp2
    expect = mask * (pg + 0.04 * (torch.exp(d) - d - 1))
    assert torch.allclose(loss, expect, atol=1e-5, rtol=1e-4)
    loss.sum().backward()
    expect.sum().backward()
    assert torch.allclose(lp.grad, lp2.grad, atol=1e-5, rtol=1e-4)


def test_rollout_engine_with_cuda_graph_matches_eager():
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.ops import native
    from ironcore_b200.parallel import mesh
    from ironcore_b200.rl import RolloutEngine

    mesh.destroy_model_parallel()
    cfg = tiny_config("qwen", d_model=256, d_ffn=512, num_layers=2, num_attention_heads=4, num_attention_groups=2,
                      head_dim=128, max_seq_len=128, max_position_embeddings=128, precision="bf16", vocab_size=1024,
                      qkv_bias=True)
    cfg.data.vocab_size = 1024
    validate_config(cfg)
    torch.manual_seed(3)
    model = LanguageModel(cfg, device=torch.device("cuda")).cuda().eval()
    prompts = torch.randint(0, 1024, (6, 32))
    eager = RolloutEngine(model, cfg, max_seqs=6, max_seq_len=128, use_cuda_graph=False)
    t1, lp1 = eager.generate(prompts, 24, temperature=0.0)
    graph = RolloutEngine(model, cfg, max_seqs=6, max_seq_len=128, use_cuda_graph=True)
    t2, lp2 = graph.generate(prompts, 24, temperature=0.0)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(t1, t2)
    assert torch.allclose(lp1, lp2, atol=1e-3)
    # decode path agrees with the cache-less training forward on the chosen tokens' log-probs
    full = model.token_logprobs(t1[:, :-1], t1[:, 1:])[:, 31:]
    assert (full - lp1).abs().max().item() < 0.15


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gumbel_sampling_kernel(dtype):
    """One-pass sampling kernel: the reported log-prob is log_softmax at the sampled token, padded columns are
    never drawn, the same (seed, draw) reproduces the sample, and the draws follow softmax(logits / T)."""
    from ironcore_b200.rl.sampling import sample_tokens

    torch.manual_seed(4)
    s, v, valid, temp = 33, 5000, 4931, 0.7
    logits = (torch.randn(s, v, device="cuda") * 3).to(dtype)
    g1, g2 = (torch.Generator(device="cuda") for _ in range(2))
    g1.manual_seed(11), g2.manual_seed(11)
    tok, lp = sample_tokens(logits, temp, generator=g1, vocab_start=100, vocab_valid=valid)
    tok2, lp2 = sample_tokens(logits, temp, generator=g2, vocab_start=100, vocab_valid=valid)
    assert torch.equal(tok, tok2) and torch.equal(lp, lp2)
    local = tok - 100
    assert int(local.min()) >= 0 and int(local.max()) < valid
    ref = torch.log_softmax(logits.float()[:, :valid] / temp, dim=-1).gather(1, local[:, None]).squeeze(1)
    assert torch.allclose(lp, ref, atol=2e-3, rtol=1e-4), (lp - ref).abs().max().item()
    # a second draw from the same generator differs
    tok3, _ = sample_tokens(logits, temp, generator=g1, vocab_start=100, vocab_valid=valid)
    assert not torch.equal(tok, tok3)
    # distribution: 40 000 rows of the same 12 logits
    base = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -2.0, 0.2, 0.9, -0.5, 1.2, 0.0], device="cuda")
    n = 40000
    many = base.to(dtype).repeat(n, 1)
    draws, _ = sample_tokens(many, 1.0, generator=g1)
    freq = torch.bincount(draws, minlength=12).float() / n
    want = torch.softmax(base.to(dtype).float(), -1)
    sigma = torch.sqrt(want * (1 - want) / n)
    assert ((freq - want).abs() < 5 * sigma + 1e-4).all(), (freq, want)
