"""HuggingFace interop must be forward-equivalent: logits of a tiny random `transformers` model and of
the native model loaded from it agree, and an exported native model reloads into `transformers`."""

import pytest
import torch

from helpers import tiny_config

transformers = pytest.importorskip("transformers")


def _native(family, **kw):
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = tiny_config(family, **kw)
    validate_config(cfg)
    return cfg, LanguageModel(cfg).eval()


def test_architecture_aliases():
    from ironcore_b200.checkpoint.hf_interop import Architecture, detect_architecture

    assert detect_architecture("gpt2") == Architecture.GPT2
    assert detect_architecture("gpt2-small") == Architecture.GPT2
    for name in ("llama", "llama3", "mistral", "qwen2", "gemma", "something-new"):
        assert detect_architecture(name) == Architecture.LLAMA


def test_gpt2_forward_equivalence_and_roundtrip(tmp_path):
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface, load_from_huggingface

    torch.manual_seed(0)
    hcfg = transformers.GPT2Config(vocab_size=512, n_positions=32, n_embd=64, n_layer=2, n_head=4, n_inner=128,
                                   resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, activation_function="gelu")
    hf = transformers.GPT2LMHeadModel(hcfg).eval()
    cfg, model = _native("gpt2", hf_model_type="gpt2")
    load_from_huggingface(model, cfg, {k: v for k, v in hf.state_dict().items()})
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        ref = hf(ids).logits
        got = model(ids)[..., :512]
    assert torch.allclose(ref, got, atol=2e-4), (ref - got).abs().max()
    out = export_to_huggingface(model, cfg, tmp_path / "hf_gpt2")
    back = transformers.GPT2LMHeadModel.from_pretrained(out).eval()
    with torch.no_grad():
        again = back(ids).logits
    assert torch.allclose(ref, again, atol=2e-4)


@pytest.mark.parametrize("interleaved", [True, False])
def test_llama_forward_equivalence_and_roundtrip(tmp_path, interleaved):
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface, load_from_huggingface, read_hf_state_dict

    torch.manual_seed(1)
    hcfg = transformers.LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                    rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                                    attention_bias=False)
    hf = transformers.LlamaForCausalLM(hcfg).eval()
    cfg, model = _native("llama", hf_model_type="llama",
                         positional_embedding={"type": "rope", "base": 10000.0, "interleaved": interleaved})
    load_from_huggingface(model, cfg, {k: v for k, v in hf.state_dict().items()})
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        ref = hf(ids).logits
        got = model(ids)[..., :512]
    assert torch.allclose(ref, got, atol=3e-4), (ref - got).abs().max()
    out = export_to_huggingface(model, cfg, tmp_path / "hf_llama", max_shard_bytes=100_000)
    assert (out / "model.safetensors.index.json").exists()
    sd = read_hf_state_dict(out)
    for k, v in hf.state_dict().items():
        assert torch.allclose(v, sd[k], atol=1e-6), k
