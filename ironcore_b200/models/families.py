"""Model-family resolution. One unified transformer covers every family; the family name
(prefix of ``model.name``) fills in the architecture switches the user left unset.
(Behavioural reference: ironcore/models/__init__.py:14-25 — a name-prefix whitelist with no
family-specific code. The family switches below — Gemma's sqrt(d) embedding scale and
(1 + w) norm gain, Phi's parallel block / partial rotary / LM-head bias, Qwen's QKV-only
bias — follow the published architectures.)"""

from __future__ import annotations

import math

FAMILIES = ("GPT", "LLAMA", "GEMMA1", "GEMMA", "QWEN", "PHI1", "PHI2", "MISTRAL", "MOE", "DUMMY")


def family_of(name: str) -> str:
    if not name:
        raise ValueError("model.name is required (e.g. gpt2-small, llama, gemma1, qwen, phi2, dummy)")
    up = name.upper().replace("-", "").replace("_", "")
    for fam in ("GEMMA1", "GEMMA", "PHI1", "PHI2", "LLAMA", "QWEN", "MISTRAL", "GPT", "MOE", "DUMMY"):
        if up.startswith(fam):
            return "GEMMA1" if fam == "GEMMA" else fam
    raise ValueError(f"model '{name}' is not a supported family ({', '.join(FAMILIES)})")


def resolve_family_defaults(model_cfg) -> str:
    """Fill the Optional architecture switches from the family. Returns the family tag."""
    fam = family_of(model_cfg.name)
    m = model_cfg
    pe = m.positional_embedding
    if m.qkv_bias is None:
        m.qkv_bias = True if fam == "QWEN" else (not m.no_bias)
    if m.norm_weight_offset is None:
        m.norm_weight_offset = 1.0 if fam == "GEMMA1" else 0.0
    if m.embed_scale is None and fam == "GEMMA1":
        m.embed_scale = math.sqrt(m.d_model)
    if m.parallel_block is None:
        m.parallel_block = fam in ("PHI1", "PHI2")
    if pe.rotary_fraction is None:
        pe.rotary_fraction = {"PHI1": 0.5, "PHI2": 0.4}.get(fam, 1.0)
    if m.lm_head_bias is None:
        m.lm_head_bias = fam in ("PHI1", "PHI2") and not m.no_bias
    if m.num_attention_groups is None:
        m.num_attention_groups = m.num_attention_heads
    if m.head_dim is None:
        m.head_dim = m.d_model // m.num_attention_heads
    return fam
