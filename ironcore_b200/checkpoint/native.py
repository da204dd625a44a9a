"""Native checkpoints.

Layout (compatible with the reference's directory format):
  ``<model_path>/step_<N>/pytorch_model.bin``          universal: TP-merged tensors
  ``<model_path>/step_<N>/tp<r>/pytorch_model.bin``    ``operation.save_dist_ckpt``: one shard per TP rank
  ``<model_path>/latest_step.txt``, ``<model_path>/config.json`` (HuggingFace-style summary)
File content: ``{model_state_dict, optimizer_state_dict{state{name: {step, exp_avg, exp_avg_sq}},
param_groups}, lr_scheduler, step, config, hf_config}`` plus ``rng`` and ``data_cursor``.
Tensor names are the canonical un-prefixed names (a ``module.`` prefix is accepted on
load), linear weights are ``[in, out]``. In a universal checkpoint both the weights and the
optimizer moments are merged across TP ranks (column-parallel tensors along the output dim
per fused part, row-parallel along the input dim), and expert tensors across EP ranks, so a
run can resume with a different TP / EP size.
(Behavioural reference: ironcore/checkpointing/native.py:39-491.)
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..parallel import mesh
from ..parallel.tensor_parallel import shard_tensor, unshard_tensors

CKPT_NAME = "pytorch_model.bin"


class HFConfigManager:
    """HuggingFace-style ``config.json`` next to the checkpoints."""

    @staticmethod
    def get_hf_config(config) -> dict:
        m = config.model
        return {
            "model_type": m.hf_model_type or (m.name or "ironcore").lower(),
            "hidden_size": m.d_model,
            "num_hidden_layers": m.num_layers,
            "num_attention_heads": m.num_attention_heads,
            "num_key_value_heads": m.num_attention_groups or m.num_attention_heads,
            "head_dim": m.head_dim,
            "intermediate_size": m.d_ffn,
            "max_position_embeddings": m.max_position_embeddings,
            "vocab_size": m.vocab_size or config.data.vocab_size,
            "layer_norm_eps": m.ln_eps,
            "rms_norm_eps": m.ln_eps,
            "rope_theta": m.positional_embedding.base,
            "initializer_range": config.init.init_std,
            "hidden_act": m.activation_type,
            "tie_word_embeddings": not m.untie_embed,
            "architectures": [m.hf_architecture or "IronCoreForCausalLM"],
        }

    @staticmethod
    def save_hf_config(config, save_directory):
        p = Path(save_directory)
        p.mkdir(parents=True, exist_ok=True)
        (p / "config.json").write_text(json.dumps(HFConfigManager.get_hf_config(config), indent=4))

    @staticmethod
    def load_hf_config(load_directory) -> dict:
        p = Path(load_directory) / "config.json"
        if not p.exists():
            raise FileNotFoundError(f"HuggingFace config file {p} does not exist.")
        return json.loads(p.read_text())


def _base_model(model):
    """The object exposing canonical_state_dict(): the FSDP wrapper itself (it gathers shards
    around the call) or the plain language model."""
    if getattr(model, "is_fsdp_wrapper", False):
        return model
    return model.module if hasattr(model, "module") else model


def _group_gather_cpu(t: torch.Tensor, group, size: int):
    """All ranks of ``group`` get every rank's tensor (moved to CPU for merging)."""
    if size == 1:
        return [t.detach().cpu()]
    parts = [torch.empty_like(t) for _ in range(size)]
    dist.all_gather(parts, t.detach().contiguous(), group=group)
    return [p.cpu() for p in parts]


def merge_model_parallel_state(local: Dict[str, torch.Tensor], shard_info: Dict[str, tuple], expert_names=()) \
        -> Dict[str, torch.Tensor]:
    """TP (and EP) merge of a name->tensor dict. Collective: every rank of the TP / EP group
    must call it with the same key order."""
    tp_group, tp = mesh.get_tensor_model_parallel_group(), mesh.get_tensor_model_parallel_world_size()
    ep_group, ep = mesh.get_expert_model_parallel_group(), mesh.get_expert_model_parallel_world_size()
    out = {}
    for name, t in local.items():
        dim, parts = shard_info.get(name, (None, 1))
        if name in expert_names and ep > 1:
            shards = _group_gather_cpu(t, ep_group, ep)
            out[name] = torch.cat(shards, dim=0)
        elif dim is not None and tp > 1:
            shards = _group_gather_cpu(t, tp_group, tp)
            out[name] = unshard_tensors(shards, dim, parts)
        else:
            out[name] = t.detach().cpu()
    return out


def split_model_parallel_tensor(full: torch.Tensor, dim, parts, name: str, expert_names=()) -> torch.Tensor:
    tp, tp_rank = mesh.get_tensor_model_parallel_world_size(), mesh.get_tensor_model_parallel_rank()
    ep, ep_rank = mesh.get_expert_model_parallel_world_size(), mesh.get_expert_model_parallel_rank()
    if name in expert_names and ep > 1:
        return full.chunk(ep, dim=0)[ep_rank].contiguous()
    if dim is not None and tp > 1:
        return shard_tensor(full, dim, parts, tp_rank, tp)
    return full


_VOCAB_DIM = {"embedding.word_embeddings.weight": 0, "output_layer.weight": 1, "output_layer.bias": 0}


def fit_padded_vocab(name: str, full: torch.Tensor, padded_vocab: int) -> torch.Tensor:
    """The padded vocabulary size is a multiple of ``vocab_padding_unit`` x the tensor-parallel size, so a merged
    checkpoint written under one TP size can carry more or fewer padding rows than the model that resumes it.
    Padding rows hold zeros and are never addressed: cut them off or add zeros along the vocabulary dimension."""
    dim = _VOCAB_DIM.get(name)
    if dim is None or padded_vocab <= 0 or full.dim() <= dim or full.shape[dim] == padded_vocab:
        return full
    if full.shape[dim] > padded_vocab:
        return full.narrow(dim, 0, padded_vocab).contiguous()
    pad = list(full.shape)
    pad[dim] = padded_vocab - full.shape[dim]
    return torch.cat([full, full.new_zeros(pad)], dim=dim)


def _ckpt_dir(config, step: int, dist_ckpt: bool) -> Path:
    base = Path(config.trainer.model_path) / f"step_{step}"
    if dist_ckpt:
        base = base / f"tp{mesh.get_tensor_model_parallel_rank()}"
        ep = mesh.get_expert_model_parallel_world_size()
        if ep > 1:
            base = base.parent / f"tp{mesh.get_tensor_model_parallel_rank()}_ep{mesh.get_expert_model_parallel_rank()}"
    return base


def _rng_state():
    st = {"torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def save_checkpoint(config, model, optimizer=None, lr_scheduler=None, step: int = 0, data_cursor: Optional[int] = None):
    """Write a checkpoint for ``step``. Collective over the TP / EP / DP groups."""
    if not config.trainer.model_path or config.operation.no_save:
        return None
    base = _base_model(model)
    dist_ckpt = bool(config.operation.save_dist_ckpt)
    tp = mesh.get_tensor_model_parallel_world_size()
    ep = mesh.get_expert_model_parallel_world_size()
    info = base.canonical_shard_info()
    local = {k: v.detach() for k, v in base.canonical_state_dict().items()}
    expert_names = {n for n in local if ".experts_" in n}
    universal = not dist_ckpt and (tp > 1 or ep > 1)
    model_sd = merge_model_parallel_state(local, info, expert_names) if universal \
        else {k: v.cpu() for k, v in local.items()}
    opt_sd = None
    if optimizer is not None:
        opt_sd = optimizer.state_dict()
        if universal and "state" in opt_sd:
            merged_state = {}
            canon = _canonical_optimizer_state(base, opt_sd["state"])
            for key in ("exp_avg", "exp_avg_sq"):
                dev0 = next(base.parameters()).device
                flat = {n: st[key].to(dev0) for n, st in canon.items()}
                merged = merge_model_parallel_state(flat, info, expert_names)
                for n, t in merged.items():
                    merged_state.setdefault(n, {"step": canon[n]["step"]})[key] = t
            opt_sd = dict(opt_sd, state=merged_state)
        elif "state" in opt_sd:
            opt_sd = dict(opt_sd, state=_canonical_optimizer_state(base, opt_sd["state"]))
    payload = {
        "model_state_dict": model_sd,
        "optimizer_state_dict": opt_sd,
        "lr_scheduler": lr_scheduler.state_dict() if lr_scheduler is not None else None,
        "step": int(step),
        "config": config.to_dict(),
        "hf_config": HFConfigManager.get_hf_config(config),
        "rng": _rng_state(),
        "data_cursor": data_cursor,
        "tp_size": 1 if universal else tp,
        "ep_size": 1 if universal else ep,
    }
    writer = mesh.get_data_parallel_rank() == 0 and (dist_ckpt or mesh.get_tensor_model_parallel_rank() == 0)
    if ep > 1 and not dist_ckpt:
        writer = mesh.get_rank() == 0
    elif ep > 1:
        writer = mesh.get_data_parallel_rank() < ep
    path = _ckpt_dir(config, step, dist_ckpt)
    if writer:
        path.mkdir(parents=True, exist_ok=True)
        tmp = path / (CKPT_NAME + ".tmp")
        torch.save(payload, tmp)
        os.replace(tmp, path / CKPT_NAME)
    if mesh.is_rank_zero():
        root = Path(config.trainer.model_path)
        root.mkdir(parents=True, exist_ok=True)
        HFConfigManager.save_hf_config(config, root)
    if dist.is_initialized():
        dist.barrier()
    if mesh.is_rank_zero():
        # the pointer moves only after every writer finished: a crash never leaves it dangling
        (Path(config.trainer.model_path) / "latest_step.txt").write_text(str(int(step)))
    return path


def _canonical_optimizer_state(base, state: Dict[str, dict]) -> Dict[str, dict]:
    """Optimizer state keyed by internal names -> canonical names (fused qkv split into q / kv)."""
    out = {}
    for name, st in state.items():
        name = name[7:] if name.startswith("module.") else name
        if ".linear_qkv." in name:
            inner = base.module if getattr(base, "is_fsdp_wrapper", False) else base
            layer = inner.model.layers[int(name.split(".")[2])]
            qn = layer.heads_local * layer.head_dim
            q = {"step": st["step"]}
            kv = {"step": st["step"]}
            for key in ("exp_avg", "exp_avg_sq"):
                a, b = st[key].split([qn, st[key].shape[-1] - qn], dim=-1)
                q[key], kv[key] = a.contiguous(), b.contiguous()
            out[name.replace("linear_qkv", "linear_q")] = q
            out[name.replace("linear_qkv", "linear_kv")] = kv
        else:
            out[name] = st
    return out


def _internal_optimizer_state(state: Dict[str, dict]) -> Dict[str, dict]:
    out, fused = {}, {}
    for name, st in state.items():
        name = name[7:] if name.startswith("module.") else name
        if ".linear_q." in name:
            fused.setdefault(name.replace("linear_q", "linear_qkv"), {})["q"] = st
        elif ".linear_kv." in name:
            fused.setdefault(name.replace("linear_kv", "linear_qkv"), {})["kv"] = st
        else:
            out[name] = st
    for name, parts in fused.items():
        if "q" in parts and "kv" in parts:
            out[name] = {"step": parts["q"]["step"],
                         "exp_avg": torch.cat([parts["q"]["exp_avg"], parts["kv"]["exp_avg"]], dim=-1),
                         "exp_avg_sq": torch.cat([parts["q"]["exp_avg_sq"], parts["kv"]["exp_avg_sq"]], dim=-1)}
    return out


def find_latest_step(model_path) -> Optional[int]:
    root = Path(model_path)
    marker = root / "latest_step.txt"
    if marker.exists():
        try:
            return int(marker.read_text().strip())
        except ValueError:
            pass
    steps = []
    if root.exists():
        for d in root.glob("step_*"):
            try:
                steps.append(int(d.name.split("_")[1]))
            except (IndexError, ValueError):
                continue
    return max(steps) if steps else None


def load_checkpoint(config, model, optimizer=None, lr_scheduler=None, step: int = -1) -> int:
    """Restore model / optimizer / scheduler; returns the checkpoint's step or -1 when there
    is nothing to load (``model_path`` empty also disables saving)."""
    if not config.trainer.model_path:
        config.operation.no_save = True
        return -1
    if step is None or step < 0:
        found = find_latest_step(config.trainer.model_path)
        if found is None:
            return -1
        step = found
    base_dir = Path(config.trainer.model_path) / f"step_{step}"
    shard_dir = _ckpt_dir(config, step, True)
    path = shard_dir / CKPT_NAME if (shard_dir / CKPT_NAME).exists() else base_dir / CKPT_NAME
    if not path.exists():
        raise FileNotFoundError(f"checkpoint {path} does not exist")
    try:
        ckpt = torch.load(path, map_location="cpu", weights_only=False)
    except Exception as exc:
        raise RuntimeError(f"checkpoint {path} is unreadable (truncated or corrupt): {exc}") from exc
    base = _base_model(model)
    info = base.canonical_shard_info()
    own = base.canonical_state_dict()
    expert_names = {n for n in own if ".experts_" in n}
    saved_tp = int(ckpt.get("tp_size", 1))
    padded_vocab = int(getattr(base, "padded_vocab_size", None) or getattr(getattr(base, "module", None),
                                                                           "padded_vocab_size", 0) or 0)
    sharded_file = path.parent != base_dir
    if sharded_file and saved_tp != mesh.get_tensor_model_parallel_world_size():
        raise ValueError(f"distributed checkpoint was written with TP={saved_tp}, "
                         f"cannot resume with TP={mesh.get_tensor_model_parallel_world_size()}")
    new_sd = {}
    for name, t in ckpt["model_state_dict"].items():
        name = name[7:] if name.startswith("module.") else name
        if name not in own:
            continue
        if not sharded_file:
            dim, parts = info.get(name, (None, 1))
            t = fit_padded_vocab(name, t, padded_vocab)
            t = split_model_parallel_tensor(t, dim, parts, name, expert_names)
        if t.numel() != own[name].numel():
            raise ValueError(f"checkpoint tensor {name} has {t.numel()} elements, model expects {own[name].numel()}")
        new_sd[name] = t.reshape(own[name].shape)
    base.load_canonical_state_dict(new_sd, strict=False)
    if optimizer is not None and config.optim.load_checkpoint_optim_state and ckpt.get("optimizer_state_dict"):
        osd = dict(ckpt["optimizer_state_dict"])
        state = {}
        for name, st in osd.get("state", {}).items():
            name = name[7:] if name.startswith("module.") else name
            if not sharded_file:
                dim, parts = info.get(name, (None, 1))
                st = {"step": st["step"],
                      "exp_avg": split_model_parallel_tensor(fit_padded_vocab(name, st["exp_avg"], padded_vocab),
                                                             dim, parts, name, expert_names),
                      "exp_avg_sq": split_model_parallel_tensor(fit_padded_vocab(name, st["exp_avg_sq"], padded_vocab),
                                                                dim, parts, name, expert_names)}
            state[name] = st
        osd["state"] = _internal_optimizer_state(state)
        optimizer.load_state_dict(osd)
    if lr_scheduler is not None and config.optim.load_checkpoint_lr_scheduler and ckpt.get("lr_scheduler"):
        lr_scheduler.load_state_dict(ckpt["lr_scheduler"])
    rng = ckpt.get("rng")
    if rng:
        torch.set_rng_state(rng["torch"])
        if torch.cuda.is_available() and "cuda" in rng:
            try:
                torch.cuda.set_rng_state(rng["cuda"])
            except Exception:
                pass
    return int(ckpt["step"])
