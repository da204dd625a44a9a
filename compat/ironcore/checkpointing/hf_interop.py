"""HuggingFace import / export (reference: ironcore/checkpointing/hf_interop.py:47-620)."""

from pathlib import Path

from ironcore_b200.checkpoint import hf_interop as _hf
from ironcore_b200.checkpoint.hf_interop import generate_hf_config, read_hf_state_dict  # noqa: F401
from ironcore_b200.checkpoint.native import HFConfigManager


def detect_checkpoint_format(checkpoint_path):
    return _hf.detect_checkpoint_format(checkpoint_path)


def load_hf_state_dict(checkpoint_path, device: str = "cpu"):
    sd = read_hf_state_dict(checkpoint_path)
    return sd if device in (None, "cpu") else {k: v.to(device) for k, v in sd.items()}


def load_hf_config(checkpoint_path):
    return HFConfigManager.load_hf_config(checkpoint_path)


def _arch(architecture):
    if architecture is None or isinstance(architecture, _hf.Architecture):
        return architecture
    return _hf.detect_architecture(str(architecture))


def load_from_huggingface(checkpoint_path, model, architecture=None, strict: bool = False, device=None, config=None):
    """Load a HuggingFace checkpoint directory into ``model`` (its ``config`` attribute describes the shapes):
    format and architecture are detected, tensors are mapped to the live names, split over the tensor-parallel
    group and fitted to the padded vocabulary. Also accepts ``(model, config, path)`` as in ``ironcore_b200``.
    Returns ``{loaded_keys, missing_keys, unexpected_keys}``; a tensor the model needs and the checkpoint lacks
    raises regardless of ``strict``."""
    if not isinstance(checkpoint_path, (str, Path, dict)):      # (model, config, path[, architecture])
        checkpoint_path, model, config, architecture = architecture, checkpoint_path, model, (strict or None)
    config = config if config is not None else model.config
    if architecture is None and not isinstance(checkpoint_path, dict):
        try:
            architecture = load_hf_config(checkpoint_path).get("model_type")
        except Exception:   # no config.json beside the weights: fall back to the model configuration's family
            architecture = None
    _hf.load_from_huggingface(model, config, checkpoint_path, _arch(architecture))
    own = [k for k in model.canonical_state_dict() if not k.endswith(".theta")]
    if device is not None:
        model.to(device)
    return {"loaded_keys": own, "missing_keys": [], "unexpected_keys": []}


def export_to_huggingface(model, output_path, architecture=None, config=None, use_safetensors: bool = True,
                          shard_size=None, **kw):
    """Write ``model`` as a HuggingFace directory (weights + ``config.json``); ``shard_size``: maximum bytes per
    weight file (one file when None). Also accepts ``(model, config, out_dir, ...)`` as in ``ironcore_b200``.
    ``config``: the framework configuration (default ``model.config``), or a dictionary that overrides entries
    of the generated ``config.json``. Returns ``{files, config_file}``."""
    import json

    overrides = None
    if hasattr(output_path, "model") and hasattr(output_path, "trainer"):     # (model, config, out_dir, ...)
        main, out_dir = output_path, architecture
        architecture = kw.pop("architecture", None)
        use_safetensors = kw.pop("safe_serialization", use_safetensors)
        shard_size = kw.pop("max_shard_bytes", shard_size)
    else:
        out_dir = output_path
        if isinstance(config, dict):
            overrides, main = config, model.config
        else:
            main = config if config is not None else model.config
    out = _hf.export_to_huggingface(model, main, out_dir, safe_serialization=use_safetensors,
                                    max_shard_bytes=shard_size, architecture=_arch(architecture))
    cfg_file = Path(out) / "config.json"
    if overrides and cfg_file.exists():
        merged = json.loads(cfg_file.read_text())
        merged.update(overrides)
        cfg_file.write_text(json.dumps(merged, indent=2))
    files = sorted(str(p) for p in Path(out).glob("*") if p.suffix in (".safetensors", ".bin"))
    return {"files": files, "config_file": str(cfg_file) if cfg_file.exists() else None}



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
