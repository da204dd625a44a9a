"""HuggingFace interoperability: load HF checkpoints into the native layout and export back,
forward-equivalent in both directions.

Native layout: linear weights ``[in, out]`` applied as ``x @ W``; q / (k|v) as ``linear_q`` /
``linear_kv``; gated MLPs fuse (gate | up) in ``mlp.up_proj``; rotary pairs are interleaved
``(2i, 2i+1)`` unless ``positional_embedding.interleaved`` is false. Conversions therefore
transpose ``nn.Linear`` weights, split / fuse projections, permute the q / k output features
between HF's rotate-half order and the interleaved order, and pad / truncate the vocabulary.
Supported families: GPT-2 (Conv1D weights) and the Llama layout (Llama 2/3, Mistral, Qwen 2/3
with QKV bias, Gemma). Under tensor parallelism every rank converts the full tensor and keeps
its shard; export gathers the shards first.
(Behavioural reference: ironcore/checkpointing/hf_interop.py:47-616 and weight_mapping.py:35-657 —
which map names and shapes only; the mappings here are checked for forward equivalence.)
"""

from __future__ import annotations

import json
import re
from enum import Enum
from pathlib import Path
from typing import Dict, Optional

import torch

from ..parallel import mesh
from .native import merge_model_parallel_state, split_model_parallel_tensor


class Architecture(Enum):
    GPT2 = "gpt2"
    LLAMA = "llama"
    PHI = "phi"


_ALIASES = {"gpt2": Architecture.GPT2, "gpt-2": Architecture.GPT2, "gpt": Architecture.GPT2, "llama": Architecture.LLAMA,
            "llama2": Architecture.LLAMA, "llama3": Architecture.LLAMA, "mistral": Architecture.LLAMA,
            "mixtral": Architecture.LLAMA, "qwen": Architecture.LLAMA, "qwen2": Architecture.LLAMA,
            "qwen3": Architecture.LLAMA, "gemma": Architecture.LLAMA, "gemma2": Architecture.LLAMA,
            "phi": Architecture.PHI, "phi1": Architecture.PHI, "phi15": Architecture.PHI, "phi2": Architecture.PHI}


def detect_architecture(model_type: Optional[str]) -> Architecture:
    """Unknown model types are treated as the Llama layout."""
    if not model_type:
        return Architecture.LLAMA
    key = re.sub(r"[-_. ]", "", str(model_type).lower())
    key = re.sub(r"(small|medium|large|xl|\d+b|\d+m)$", "", key)
    return _ALIASES.get(key, Architecture.GPT2 if key.startswith("gpt2") else Architecture.LLAMA)


def _rope_perm(head_dim: int, to_interleaved: bool, rot_dim: Optional[int] = None) -> torch.Tensor:
    """Index permutation of one head's output features between HF rotate-half order
    (pairs (j, j + rot/2)) and interleaved order (pairs (2j, 2j + 1)) over the first ``rot_dim`` features (all of
    them by default); features beyond ``rot_dim`` (partial rotary) keep their place."""
    rot = head_dim if rot_dim is None else rot_dim
    half = rot // 2
    inter_from_hf = torch.arange(head_dim)
    inter_from_hf[0:rot:2] = torch.arange(half)
    inter_from_hf[1:rot:2] = torch.arange(half) + half
    if to_interleaved:
        return inter_from_hf
    inv = torch.empty_like(inter_from_hf)
    inv[inter_from_hf] = torch.arange(head_dim)
    return inv


def _permute_heads(w_in_out: torch.Tensor, heads: int, head_dim: int, to_interleaved: bool,
                   rot_dim: Optional[int] = None) -> torch.Tensor:
    """Permute the output features (last dim) of a [in, heads*hd] weight or a [heads*hd] bias."""
    perm = _rope_perm(head_dim, to_interleaved, rot_dim)
    shape = w_in_out.shape
    x = w_in_out.reshape(*shape[:-1], heads, head_dim)
    return x[..., perm].reshape(shape)


class WeightMapper:
    """Name and layout mapping between HF state dicts and the canonical native state dict."""

    def __init__(self, architecture: Architecture, num_layers: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 gated_mlp: bool = True, interleaved_rope: bool = True, tie_embeddings: bool = False,
                 rot_dim: Optional[int] = None):
        self.arch, self.L = architecture, num_layers
        self.h, self.g, self.hd = num_heads, num_kv_heads, head_dim
        self.gated, self.interleaved, self.tied = gated_mlp, interleaved_rope, tie_embeddings
        self.rot = rot_dim if rot_dim is not None else head_dim     # rotated features per head (partial rotary)

    @classmethod
    def from_config(cls, config, architecture: Optional[Architecture] = None):
        m = config.model
        from ..layers.activations import is_glu

        arch = architecture or detect_architecture(m.hf_model_type or m.name)
        rope = m.positional_embedding.type.lower() == "rope"
        hd = m.head_dim or m.d_model // m.num_attention_heads
        rot = int(hd * float(m.positional_embedding.rotary_fraction or 1.0))
        return cls(arch, m.num_layers, m.num_attention_heads, m.num_attention_groups or m.num_attention_heads,
                   hd, is_glu(m.activation_type), bool(m.positional_embedding.interleaved) and rope,
                   not m.untie_embed, rot_dim=rot - rot % 2)

    # ------------------------------------------------------------------ HF -> native
    def hf_to_native(self, hf: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.arch == Architecture.PHI:
            return self._phi_in(hf)
        return self._gpt2_in(hf) if self.arch == Architecture.GPT2 else self._llama_in(hf)

    # Phi-1 / 1.5 / 2: one LayerNorm feeding attention and MLP in parallel, biases everywhere, a plain (ungated)
    # MLP ``fc1`` / ``fc2``, the attention output projection called ``dense``, ``final_layernorm`` and an LM head
    # with a bias; rotary on the first ``rot_dim`` features of every head.
    def _phi_in(self, hf):
        pre = "model." if any(k.startswith("model.") for k in hf) else ""
        out = {"embedding.word_embeddings.weight": hf[pre + "embed_tokens.weight"],
               "output_layernorm.layernorm.weight": hf[pre + "final_layernorm.weight"],
               "output_layernorm.layernorm.bias": hf[pre + "final_layernorm.bias"]}
        for i in range(self.L):
            p, q = f"{pre}layers.{i}.", f"model.layers.{i}."
            w = {n: hf[p + f"self_attn.{n}_proj.weight"].t() for n in "qkv"}
            b = {n: hf[p + f"self_attn.{n}_proj.bias"] for n in "qkv"}
            if self.interleaved:
                w["q"], b["q"] = (_permute_heads(t, self.h, self.hd, True, self.rot) for t in (w["q"], b["q"]))
                w["k"], b["k"] = (_permute_heads(t, self.g, self.hd, True, self.rot) for t in (w["k"], b["k"]))
            out[q + "linear_q.weight"], out[q + "linear_q.bias"] = w["q"], b["q"]
            out[q + "linear_kv.weight"] = torch.cat([w["k"], w["v"]], dim=1)
            out[q + "linear_kv.bias"] = torch.cat([b["k"], b["v"]])
            out[q + "attn_output.weight"], out[q + "attn_output.bias"] = hf[p + "self_attn.dense.weight"].t(), hf[p + "self_attn.dense.bias"]
            out[q + "input_layernorm.layernorm.weight"] = hf[p + "input_layernorm.weight"]
            out[q + "input_layernorm.layernorm.bias"] = hf[p + "input_layernorm.bias"]
            out[q + "mlp.up_proj.weight"], out[q + "mlp.up_proj.bias"] = hf[p + "mlp.fc1.weight"].t(), hf[p + "mlp.fc1.bias"]
            out[q + "mlp.down_proj.weight"], out[q + "mlp.down_proj.bias"] = hf[p + "mlp.fc2.weight"].t(), hf[p + "mlp.fc2.bias"]
        if not self.tied:
            out["output_layer.weight"] = hf["lm_head.weight"].t()
            if "lm_head.bias" in hf:
                out["output_layer.bias"] = hf["lm_head.bias"]
        return {k: v.contiguous() for k, v in out.items()}

    def _phi_out(self, sd):
        out = {"model.embed_tokens.weight": sd["embedding.word_embeddings.weight"],
               "model.final_layernorm.weight": sd["output_layernorm.layernorm.weight"],
               "model.final_layernorm.bias": sd["output_layernorm.layernorm.bias"]}
        for i in range(self.L):
            p, q = f"model.layers.{i}.", f"model.layers.{i}."
            wq, bq = sd[q + "linear_q.weight"], sd[q + "linear_q.bias"]
            (wk, wv), (bk, bv) = sd[q + "linear_kv.weight"].chunk(2, dim=1), sd[q + "linear_kv.bias"].chunk(2)
            if self.interleaved:
                wq, bq = (_permute_heads(t, self.h, self.hd, False, self.rot) for t in (wq, bq))
                wk, bk = (_permute_heads(t, self.g, self.hd, False, self.rot) for t in (wk, bk))
            for n, w_, b_ in (("q", wq, bq), ("k", wk, bk), ("v", wv, bv)):
                out[p + f"self_attn.{n}_proj.weight"], out[p + f"self_attn.{n}_proj.bias"] = w_.t(), b_
            out[p + "self_attn.dense.weight"], out[p + "self_attn.dense.bias"] = sd[q + "attn_output.weight"].t(), sd[q + "attn_output.bias"]
            out[p + "input_layernorm.weight"] = sd[q + "input_layernorm.layernorm.weight"]
            out[p + "input_layernorm.bias"] = sd[q + "input_layernorm.layernorm.bias"]
            out[p + "mlp.fc1.weight"], out[p + "mlp.fc1.bias"] = sd[q + "mlp.up_proj.weight"].t(), sd[q + "mlp.up_proj.bias"]
            out[p + "mlp.fc2.weight"], out[p + "mlp.fc2.bias"] = sd[q + "mlp.down_proj.weight"].t(), sd[q + "mlp.down_proj.bias"]
        out["lm_head.weight"] = sd["output_layer.weight"].t() if "output_layer.weight" in sd \
            else sd["embedding.word_embeddings.weight"]
        if "output_layer.bias" in sd:
            out["lm_head.bias"] = sd["output_layer.bias"]
        return {k: v.contiguous() for k, v in out.items()}

    def _gpt2_in(self, hf):
        g = lambda k: hf[k] if k in hf else hf["transformer." + k]
        has = lambda k: (k in hf) or ("transformer." + k in hf)
        out = {"embedding.word_embeddings.weight": g("wte.weight"),
               "embedding.position_embedding.weight": g("wpe.weight"),
               "output_layernorm.layernorm.weight": g("ln_f.weight"), "output_layernorm.layernorm.bias": g("ln_f.bias")}
        d = g("wte.weight").shape[1]
        for i in range(self.L):
            p, q = f"h.{i}.", f"model.layers.{i}."
            ca_w, ca_b = g(p + "attn.c_attn.weight"), g(p + "attn.c_attn.bias")   # Conv1D: already [in, out]
            out[q + "linear_q.weight"], out[q + "linear_kv.weight"] = ca_w[:, :d], ca_w[:, d:]
            out[q + "linear_q.bias"], out[q + "linear_kv.bias"] = ca_b[:d], ca_b[d:]
            out[q + "attn_output.weight"], out[q + "attn_output.bias"] = g(p + "attn.c_proj.weight"), g(p + "attn.c_proj.bias")
            out[q + "input_layernorm.layernorm.weight"], out[q + "input_layernorm.layernorm.bias"] = g(p + "ln_1.weight"), g(p + "ln_1.bias")
            out[q + "post_attn_layernorm.layernorm.weight"], out[q + "post_attn_layernorm.layernorm.bias"] = g(p + "ln_2.weight"), g(p + "ln_2.bias")
            out[q + "mlp.up_proj.weight"], out[q + "mlp.up_proj.bias"] = g(p + "mlp.c_fc.weight"), g(p + "mlp.c_fc.bias")
            out[q + "mlp.down_proj.weight"], out[q + "mlp.down_proj.bias"] = g(p + "mlp.c_proj.weight"), g(p + "mlp.c_proj.bias")
        if not self.tied and has("lm_head.weight"):
            out["output_layer.weight"] = hf["lm_head.weight"].t()
        return {k: v.contiguous() for k, v in out.items()}

    @staticmethod
    def _moe_in(hf, p: str):
        """Tensors of a mixture-of-experts layer under the native names (without the layer prefix): ``mlp.router.weight``
        [E, d], ``mlp.experts_up`` [E, d, 2f] (activated half first), ``mlp.experts_down`` [E, f, d] and, for the
        Qwen-MoE layout, the shared expert and its gate; None for a dense layer. Reads the per-expert names of
        checkpoints on disk (Mixtral: ``block_sparse_moe.gate``, ``experts.N.w1 / w3 / w2``; Qwen-MoE:
        ``mlp.experts.N.gate_proj / up_proj / down_proj``) and the stacked form that ``transformers`` keeps in
        memory (``mlp.gate``, ``mlp.experts.gate_up_proj`` / ``down_proj``)."""
        out = {}
        if p + "mlp.experts.gate_up_proj" in hf:
            out["mlp.router.weight"] = hf[p + "mlp.gate.weight"]
            out["mlp.experts_up"] = hf[p + "mlp.experts.gate_up_proj"].transpose(1, 2)
            out["mlp.experts_down"] = hf[p + "mlp.experts.down_proj"].transpose(1, 2)
        else:
            for gate, fmt, (n1, n3, n2) in (("block_sparse_moe.gate.weight", "block_sparse_moe.experts.{}.", ("w1", "w3", "w2")),
                                            ("mlp.gate.weight", "mlp.experts.{}.", ("gate_proj", "up_proj", "down_proj"))):
                if p + gate in hf and p + fmt.format(0) + n1 + ".weight" in hf:
                    ups, downs, e = [], [], 0
                    while p + fmt.format(e) + n1 + ".weight" in hf:
                        ep = p + fmt.format(e)
                        ups.append(torch.cat([hf[ep + n1 + ".weight"].t(), hf[ep + n3 + ".weight"].t()], dim=1))
                        downs.append(hf[ep + n2 + ".weight"].t())
                        e += 1
                    out["mlp.router.weight"] = hf[p + gate]
                    out["mlp.experts_up"], out["mlp.experts_down"] = torch.stack(ups), torch.stack(downs)
                    break
        if not out:
            return None
        if p + "mlp.shared_expert.up_proj.weight" in hf:
            out["mlp.shared.up_proj.weight"] = torch.cat([hf[p + "mlp.shared_expert.gate_proj.weight"].t(),
                                                          hf[p + "mlp.shared_expert.up_proj.weight"].t()], dim=1)
            out["mlp.shared.down_proj.weight"] = hf[p + "mlp.shared_expert.down_proj.weight"].t()
            if p + "mlp.shared_expert_gate.weight" in hf:
                out["mlp.shared_gate.weight"] = hf[p + "mlp.shared_expert_gate.weight"]
        return out

    def _llama_in(self, hf):
        pre = "model." if any(k.startswith("model.") for k in hf) else ""
        out = {"embedding.word_embeddings.weight": hf[pre + "embed_tokens.weight"],
               "output_layernorm.layernorm.weight": hf[pre + "norm.weight"]}
        for i in range(self.L):
            p, q = f"{pre}layers.{i}.", f"model.layers.{i}."
            wq = hf[p + "self_attn.q_proj.weight"].t()
            wk = hf[p + "self_attn.k_proj.weight"].t()
            wv = hf[p + "self_attn.v_proj.weight"].t()
            if self.interleaved:
                wq = _permute_heads(wq, self.h, self.hd, True, self.rot)
                wk = _permute_heads(wk, self.g, self.hd, True, self.rot)
            out[q + "linear_q.weight"] = wq
            out[q + "linear_kv.weight"] = torch.cat([wk, wv], dim=1)
            if p + "self_attn.q_proj.bias" in hf:
                bq, bk, bv = (hf[p + f"self_attn.{n}_proj.bias"] for n in "qkv")
                if self.interleaved:
                    bq = _permute_heads(bq, self.h, self.hd, True, self.rot)
                    bk = _permute_heads(bk, self.g, self.hd, True, self.rot)
                out[q + "linear_q.bias"] = bq
                out[q + "linear_kv.bias"] = torch.cat([bk, bv])
            out[q + "attn_output.weight"] = hf[p + "self_attn.o_proj.weight"].t()
            out[q + "input_layernorm.layernorm.weight"] = hf[p + "input_layernorm.weight"]
            out[q + "post_attn_layernorm.layernorm.weight"] = hf[p + "post_attention_layernorm.weight"]
            moe = self._moe_in(hf, p)
            if moe is not None:
                out.update({q + name: t for name, t in moe.items()})
                continue
            up = hf[p + "mlp.up_proj.weight"].t()
            if self.gated:
                up = torch.cat([hf[p + "mlp.gate_proj.weight"].t(), up], dim=1)   # (f | g): act(f) * g, f = gate
            out[q + "mlp.up_proj.weight"] = up
            out[q + "mlp.down_proj.weight"] = hf[p + "mlp.down_proj.weight"].t()
        if not self.tied:
            head = hf.get("lm_head.weight", hf[pre + "embed_tokens.weight"])
            out["output_layer.weight"] = head.t()
        return {k: v.contiguous() for k, v in out.items()}

    # ------------------------------------------------------------------ native -> HF
    def native_to_hf(self, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.arch == Architecture.PHI:
            return self._phi_out(sd)
        return self._gpt2_out(sd) if self.arch == Architecture.GPT2 else self._llama_out(sd)

    def _gpt2_out(self, sd):
        out = {"transformer.wte.weight": sd["embedding.word_embeddings.weight"],
               "transformer.wpe.weight": sd["embedding.position_embedding.weight"],
               "transformer.ln_f.weight": sd["output_layernorm.layernorm.weight"],
               "transformer.ln_f.bias": sd["output_layernorm.layernorm.bias"]}
        for i in range(self.L):
            p, q = f"transformer.h.{i}.", f"model.layers.{i}."
            out[p + "attn.c_attn.weight"] = torch.cat([sd[q + "linear_q.weight"], sd[q + "linear_kv.weight"]], dim=1)
            out[p + "attn.c_attn.bias"] = torch.cat([sd[q + "linear_q.bias"], sd[q + "linear_kv.bias"]])
            out[p + "attn.c_proj.weight"], out[p + "attn.c_proj.bias"] = sd[q + "attn_output.weight"], sd[q + "attn_output.bias"]
            out[p + "ln_1.weight"], out[p + "ln_1.bias"] = sd[q + "input_layernorm.layernorm.weight"], sd[q + "input_layernorm.layernorm.bias"]
            out[p + "ln_2.weight"], out[p + "ln_2.bias"] = sd[q + "post_attn_layernorm.layernorm.weight"], sd[q + "post_attn_layernorm.layernorm.bias"]
            out[p + "mlp.c_fc.weight"], out[p + "mlp.c_fc.bias"] = sd[q + "mlp.up_proj.weight"], sd[q + "mlp.up_proj.bias"]
            out[p + "mlp.c_proj.weight"], out[p + "mlp.c_proj.bias"] = sd[q + "mlp.down_proj.weight"], sd[q + "mlp.down_proj.bias"]
        out["lm_head.weight"] = sd["output_layer.weight"].t() if "output_layer.weight" in sd \
            else sd["embedding.word_embeddings.weight"]
        return {k: v.contiguous() for k, v in out.items()}

    def _llama_out(self, sd):
        out = {"model.embed_tokens.weight": sd["embedding.word_embeddings.weight"],
               "model.norm.weight": sd["output_layernorm.layernorm.weight"]}
        for i in range(self.L):
            p, q = f"model.layers.{i}.", f"model.layers.{i}."
            wq = sd[q + "linear_q.weight"]
            wk, wv = sd[q + "linear_kv.weight"].chunk(2, dim=1)
            if self.interleaved:
                wq = _permute_heads(wq, self.h, self.hd, False, self.rot)
                wk = _permute_heads(wk, self.g, self.hd, False, self.rot)
            out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"] = wq.t(), wk.t()
            out[p + "self_attn.v_proj.weight"] = wv.t()
            if q + "linear_q.bias" in sd:
                bq = sd[q + "linear_q.bias"]
                bk, bv = sd[q + "linear_kv.bias"].chunk(2)
                if self.interleaved:
                    bq = _permute_heads(bq, self.h, self.hd, False, self.rot)
                    bk = _permute_heads(bk, self.g, self.hd, False, self.rot)
                out[p + "self_attn.q_proj.bias"], out[p + "self_attn.k_proj.bias"], out[p + "self_attn.v_proj.bias"] = bq, bk, bv
            out[p + "self_attn.o_proj.weight"] = sd[q + "attn_output.weight"].t()
            out[p + "input_layernorm.weight"] = sd[q + "input_layernorm.layernorm.weight"]
            out[p + "post_attention_layernorm.weight"] = sd[q + "post_attn_layernorm.layernorm.weight"]
            if q + "mlp.experts_up" in sd:
                ups, downs = sd[q + "mlp.experts_up"], sd[q + "mlp.experts_down"]
                if q + "mlp.shared.up_proj.weight" in sd:
                    # Qwen-MoE names on disk: gate / up / down per expert, one shared expert and its gate
                    out[p + "mlp.gate.weight"] = sd[q + "mlp.router.weight"]
                    names, fmt = ("gate_proj", "up_proj", "down_proj"), p + "mlp.experts.{}."
                    g, u = sd[q + "mlp.shared.up_proj.weight"].chunk(2, dim=1)
                    out[p + "mlp.shared_expert.gate_proj.weight"], out[p + "mlp.shared_expert.up_proj.weight"] = g.t(), u.t()
                    out[p + "mlp.shared_expert.down_proj.weight"] = sd[q + "mlp.shared.down_proj.weight"].t()
                    if q + "mlp.shared_gate.weight" in sd:
                        out[p + "mlp.shared_expert_gate.weight"] = sd[q + "mlp.shared_gate.weight"]
                else:
                    # Mixtral names on disk: one gate, w1 (activated) / w3 / w2 per expert
                    out[p + "block_sparse_moe.gate.weight"] = sd[q + "mlp.router.weight"]
                    names, fmt = ("w1", "w3", "w2"), p + "block_sparse_moe.experts.{}."
                for e in range(ups.shape[0]):
                    w1, w3 = ups[e].chunk(2, dim=1)
                    ep = fmt.format(e)
                    out[ep + names[0] + ".weight"], out[ep + names[1] + ".weight"] = w1.t(), w3.t()
                    out[ep + names[2] + ".weight"] = downs[e].t()
                continue
            up = sd[q + "mlp.up_proj.weight"]
            if self.gated:
                gate, up = up.chunk(2, dim=1)
                out[p + "mlp.gate_proj.weight"] = gate.t()
            out[p + "mlp.up_proj.weight"] = up.t()
            out[p + "mlp.down_proj.weight"] = sd[q + "mlp.down_proj.weight"].t()
        out["lm_head.weight"] = sd["output_layer.weight"].t() if "output_layer.weight" in sd \
            else sd["embedding.word_embeddings.weight"]
        return {k: v.contiguous() for k, v in out.items()}


# ---------------------------------------------------------------------- file formats
def detect_checkpoint_format(path) -> Dict[str, object]:
    """{'format': 'safetensors'|'pytorch', 'sharded': bool, 'files': [...]} for an HF model directory."""
    p = Path(path)
    for fmt, single, index in (("safetensors", "model.safetensors", "model.safetensors.index.json"),
                               ("pytorch", "pytorch_model.bin", "pytorch_model.bin.index.json")):
        if (p / index).exists():
            files = sorted(set(json.loads((p / index).read_text())["weight_map"].values()))
            return {"format": fmt, "sharded": True, "files": [p / f for f in files]}
        if (p / single).exists():
            return {"format": fmt, "sharded": False, "files": [p / single]}
    raise FileNotFoundError(f"no HuggingFace checkpoint found in {p}")


def read_hf_state_dict(path) -> Dict[str, torch.Tensor]:
    info = detect_checkpoint_format(path)
    sd: Dict[str, torch.Tensor] = {}
    for f in info["files"]:
        if info["format"] == "safetensors":
            from safetensors.torch import load_file

            sd.update(load_file(str(f)))
        else:
            sd.update(torch.load(f, map_location="cpu", weights_only=True))
    return sd


def _fit_vocab(t: torch.Tensor, rows: int, dim: int = 0) -> torch.Tensor:
    cur = t.shape[dim]
    if cur == rows:
        return t
    if cur > rows:
        return t.narrow(dim, 0, rows)
    pad_shape = list(t.shape)
    pad_shape[dim] = rows - cur
    return torch.cat([t, torch.zeros(pad_shape, dtype=t.dtype)], dim=dim)


def load_from_huggingface(model, config, path, architecture: Optional[Architecture] = None) -> None:
    """Load an HF checkpoint directory (or a state dict) into ``model`` (a LanguageModel)."""
    hf = read_hf_state_dict(path) if not isinstance(path, dict) else path
    mapper = WeightMapper.from_config(config, architecture)
    native = mapper.hf_to_native(hf)
    padded = model.padded_vocab_size
    native["embedding.word_embeddings.weight"] = _fit_vocab(native["embedding.word_embeddings.weight"], padded, 0)
    if "output_layer.weight" in native:
        native["output_layer.weight"] = _fit_vocab(native["output_layer.weight"], padded, 1)
    info = model.canonical_shard_info()
    own = model.canonical_state_dict()
    experts = [n for n in own if n.endswith(("experts_up", "experts_down"))]    # split over the expert-parallel group
    sd = {}
    for name, t in native.items():
        if name not in own:
            continue
        dim, parts = info.get(name, (None, 1))
        t = split_model_parallel_tensor(t, dim, parts, name, expert_names=experts)
        sd[name] = t.to(own[name].dtype).reshape(own[name].shape)
    missing = [k for k in own if k not in sd and not k.endswith(".theta")]
    if missing:
        raise KeyError(f"HF checkpoint lacks tensors for: {missing[:5]}{'...' if len(missing) > 5 else ''}")
    model.load_canonical_state_dict(sd, strict=False)


def generate_hf_config(config) -> dict:
    m = config.model
    arch = detect_architecture(m.hf_model_type or m.name)
    vocab = m.vocab_size or config.data.vocab_size
    if arch == Architecture.GPT2:
        return {"model_type": "gpt2", "architectures": [m.hf_architecture or "GPT2LMHeadModel"], "vocab_size": vocab,
                "n_positions": m.max_position_embeddings, "n_embd": m.d_model, "n_layer": m.num_layers,
                "n_head": m.num_attention_heads, "n_inner": m.d_ffn, "activation_function": "gelu",
                "layer_norm_epsilon": m.ln_eps, "resid_pdrop": 0.0, "embd_pdrop": 0.0, "attn_pdrop": 0.0,
                "tie_word_embeddings": not m.untie_embed}
    if arch == Architecture.PHI:
        return {"model_type": "phi", "architectures": [m.hf_architecture or "PhiForCausalLM"], "vocab_size": vocab,
                "hidden_size": m.d_model, "intermediate_size": m.d_ffn, "num_hidden_layers": m.num_layers,
                "num_attention_heads": m.num_attention_heads,
                "num_key_value_heads": m.num_attention_groups or m.num_attention_heads, "hidden_act": "gelu_new",
                "max_position_embeddings": m.max_position_embeddings, "layer_norm_eps": m.ln_eps,
                "rope_theta": float(m.positional_embedding.base),
                "partial_rotary_factor": float(m.positional_embedding.rotary_fraction or 1.0),
                "resid_pdrop": 0.0, "embd_pdrop": 0.0, "attention_dropout": 0.0, "qk_layernorm": False,
                "tie_word_embeddings": not m.untie_embed}
    if m.moe.num_experts > 0 and m.moe.num_shared_experts:
        if not m.moe.shared_expert_gate or m.moe.layer_freq != 1 or not m.qkv_bias:
            raise ValueError("a model with shared experts exports in the Qwen-MoE layout: every layer a mixture of "
                             "experts, model.moe.shared_expert_gate on, biases on q / k / v")
        return {"model_type": "qwen2_moe", "architectures": [m.hf_architecture or "Qwen2MoeForCausalLM"],
                "vocab_size": vocab, "hidden_size": m.d_model, "intermediate_size": m.d_ffn,
                "moe_intermediate_size": m.moe.expert_d_ffn or m.d_ffn,
                "shared_expert_intermediate_size": (m.moe.shared_expert_d_ffn or m.moe.expert_d_ffn or m.d_ffn)
                * m.moe.num_shared_experts,
                "num_hidden_layers": m.num_layers, "num_attention_heads": m.num_attention_heads,
                "num_key_value_heads": m.num_attention_groups or m.num_attention_heads, "hidden_act": "silu",
                "max_position_embeddings": m.max_position_embeddings, "rms_norm_eps": m.ln_eps,
                "rope_theta": float(m.positional_embedding.base), "num_experts": m.moe.num_experts,
                "num_experts_per_tok": m.moe.top_k, "norm_topk_prob": bool(m.moe.normalize_topk),
                "decoder_sparse_step": 1, "mlp_only_layers": [], "router_aux_loss_coef": m.moe.aux_loss_coeff,
                "use_sliding_window": False, "tie_word_embeddings": not m.untie_embed}
    if m.moe.num_experts > 0:
        if not m.moe.normalize_topk or m.moe.layer_freq != 1:
            raise ValueError("a model without shared experts exports in the Mixtral layout: every layer a mixture "
                             "of experts, model.moe.normalize_topk on")
        return {"model_type": "mixtral", "architectures": [m.hf_architecture or "MixtralForCausalLM"],
                "vocab_size": vocab, "hidden_size": m.d_model, "intermediate_size": m.moe.expert_d_ffn or m.d_ffn,
                "num_hidden_layers": m.num_layers, "num_attention_heads": m.num_attention_heads,
                "num_key_value_heads": m.num_attention_groups or m.num_attention_heads, "head_dim": m.head_dim,
                "hidden_act": "silu", "max_position_embeddings": m.max_position_embeddings, "rms_norm_eps": m.ln_eps,
                "rope_theta": float(m.positional_embedding.base), "num_local_experts": m.moe.num_experts,
                "num_experts_per_tok": m.moe.top_k, "router_aux_loss_coef": m.moe.aux_loss_coeff,
                "sliding_window": None, "tie_word_embeddings": not m.untie_embed}
    from ..layers.activations import canonical_activation

    act = {"swiglu": "silu", "geglu": "gelu_pytorch_tanh", "geglu_erf": "gelu", "reglu": "relu"}.get(
        canonical_activation(m.activation_type), "silu")
    return {"model_type": m.hf_model_type or "llama", "architectures": [m.hf_architecture or "LlamaForCausalLM"],
            "vocab_size": vocab, "hidden_size": m.d_model, "intermediate_size": m.d_ffn,
            "num_hidden_layers": m.num_layers, "num_attention_heads": m.num_attention_heads,
            "num_key_value_heads": m.num_attention_groups or m.num_attention_heads, "head_dim": m.head_dim,
            "hidden_act": act, "hidden_activation": act,     # (Gemma reads the second name)
            "max_position_embeddings": m.max_position_embeddings, "rms_norm_eps": m.ln_eps,
            "rope_theta": float(m.positional_embedding.base), "tie_word_embeddings": not m.untie_embed,
            "attention_bias": bool(m.qkv_bias), "mlp_bias": False}


def export_to_huggingface(model, config, out_dir, safe_serialization: bool = True,
                          max_shard_bytes: Optional[int] = None, architecture: Optional[Architecture] = None) -> Path:
    """Write an HF-loadable directory (config.json + weights, optionally sharded with an index).
    Collective over the TP group; rank 0 writes."""
    base = model
    local = {k: v.detach() for k, v in base.canonical_state_dict().items()}
    experts = [n for n in local if n.endswith(("experts_up", "experts_down"))]   # gathered over the expert-parallel group
    merged = merge_model_parallel_state(local, base.canonical_shard_info(), expert_names=experts)
    vocab = config.model.vocab_size or config.data.vocab_size
    merged["embedding.word_embeddings.weight"] = _fit_vocab(merged["embedding.word_embeddings.weight"], vocab, 0)
    if "output_layer.weight" in merged:
        merged["output_layer.weight"] = _fit_vocab(merged["output_layer.weight"], vocab, 1)
    mapper = WeightMapper.from_config(config, architecture)
    hf = {k: v.contiguous() for k, v in mapper.native_to_hf(merged).items()}
    if not config.model.untie_embed:
        hf.pop("lm_head.weight", None)
    out = Path(out_dir)
    if mesh.is_rank_zero():
        out.mkdir(parents=True, exist_ok=True)
        (out / "config.json").write_text(json.dumps(generate_hf_config(config), indent=2))
        ext = "safetensors" if safe_serialization else "bin"
        stem = "model" if safe_serialization else "pytorch_model"

        def save(sd, path):
            if safe_serialization:
                from safetensors.torch import save_file

                save_file({k: v.clone() for k, v in sd.items()}, str(path), metadata={"format": "pt"})
            else:
                torch.save(sd, path)

        if not max_shard_bytes:
            save(hf, out / f"{stem}.{ext}")
        else:
            shards, cur, size = [], {}, 0
            for k, v in hf.items():
                nb = v.numel() * v.element_size()
                if cur and size + nb > max_shard_bytes:
                    shards.append(cur)
                    cur, size = {}, 0
                cur[k] = v
                size += nb
            if cur:
                shards.append(cur)
            weight_map = {}
            for i, sh in enumerate(shards):
                fname = f"{stem}-{i + 1:05d}-of-{len(shards):05d}.{ext}"
                save(sh, out / fname)
                weight_map.update({k: fname for k in sh})
            total = sum(v.numel() * v.element_size() for v in hf.values())
            (out / f"{stem}.{ext}.index.json").write_text(json.dumps({"metadata": {"total_size": total},
                                                                      "weight_map": weight_map}, indent=2))
    return out
