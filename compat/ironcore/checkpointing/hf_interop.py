"""HuggingFace import / export (reference: ironcore/checkpointing/hf_interop.py:47-620)."""

from ironcore_b200.checkpoint.hf_interop import (detect_checkpoint_format, export_to_huggingface,  # noqa: F401
                                                 generate_hf_config, load_from_huggingface, read_hf_state_dict)
from ironcore_b200.checkpoint.native import HFConfigManager

load_hf_state_dict = read_hf_state_dict
load_hf_config = HFConfigManager.load_hf_config


def _generate_hf_config(model, architecture: str, num_layers: int) -> dict:
    """``config.json`` contents for ``model``: from its configuration object when it carries one, otherwise from
    the shape of its word-embedding table (reference: hf_interop.py:561-616)."""
    config = getattr(model, "config", None)
    if config is not None and hasattr(config, "model") and hasattr(config, "trainer"):
        out = generate_hf_config(config)
        out["n_layer" if out["model_type"] == "gpt2" else "num_hidden_layers"] = num_layers
        return out
    vocab = hidden = heads = None
    for name, p in model.named_parameters():
        if "embedding" in name and name.endswith("weight") and p.dim() == 2:
            vocab, hidden = p.shape
            break
    for mod in model.modules():
        if hasattr(mod, "num_attention_heads"):
            heads = mod.num_attention_heads
            break
    if architecture.lower() in ("gpt2", "gpt"):
        return {"model_type": "gpt2", "architectures": ["GPT2LMHeadModel"], "vocab_size": vocab or 50257,
                "n_embd": hidden or 768, "n_layer": num_layers, "n_head": heads or 12, "n_positions": 1024,
                "activation_function": "gelu_new"}
    hidden = hidden or 4096
    return {"model_type": architecture.lower(), "architectures": [f"{architecture.title()}ForCausalLM"],
            "vocab_size": vocab or 32000, "hidden_size": hidden, "num_hidden_layers": num_layers,
            "num_attention_heads": heads or 32, "intermediate_size": 4 * hidden, "max_position_embeddings": 4096,
            "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
