"""YAML / CLI / environment loading and validation of :class:`MainConfig`.

Precedence: dataclass defaults < YAML file < ``--<field>`` command-line overrides <
rank variables from the environment. A group in the YAML file is either an inline
mapping or a string naming ``<dir of main file>/<group>/<name>.yaml`` (the group's
``name`` is then recorded). ``${VAR}`` is interpolated from the environment and lists
of single-key mappings are merged into one mapping.
(Behavioural reference: ironcore/config/__init__.py:47-140, 371-431, 463-515;
ironcore/utils.py:24-82.)
"""

from __future__ import annotations

import argparse
import os
import re
import typing
from dataclasses import fields, is_dataclass
from pathlib import Path
from typing import Any, Dict, Optional, Sequence

import yaml

from .schema import GROUPS, BaseConfig, MainConfig

_ENV_PATTERN = re.compile(r"\$\{(\w+)\}")


def load_dotenv(path: str = ".env") -> None:
    """Minimal .env reader (KEY=VALUE lines); existing variables win."""
    p = Path(path)
    if not p.exists():
        return
    for line in p.read_text().splitlines():
        line = line.strip()
        if not line or line.startswith("#") or "=" not in line:
            continue
        k, v = line.split("=", 1)
        os.environ.setdefault(k.strip(), v.strip().strip('"').strip("'"))


def _interpolate(node: Any) -> Any:
    if isinstance(node, str):
        return _ENV_PATTERN.sub(lambda m: os.environ.get(m.group(1), ""), node)
    if isinstance(node, dict):
        return {k: _interpolate(v) for k, v in node.items()}
    if isinstance(node, list):
        return [_interpolate(v) for v in node]
    return node


def _merge_single_key_lists(node: Any) -> Any:
    if isinstance(node, dict):
        return {k: _merge_single_key_lists(v) for k, v in node.items()}
    if isinstance(node, list):
        if node and all(isinstance(it, dict) for it in node):
            merged: Dict[str, Any] = {}
            for it in node:
                merged.update(it)
            return {k: _merge_single_key_lists(v) for k, v in merged.items()}
        return node
    return node


def load_yaml_config(path, merge_lists: bool = True) -> Dict[str, Any]:
    """Read a YAML file with ``${ENV}`` interpolation and (for trainer configs) merging of
    lists of single-key mappings; dataset YAMLs keep their lists (``merge_lists=False``)."""
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"Config file not found: {p}")
    try:
        raw = yaml.safe_load(p.read_text(encoding="utf-8")) or {}
    except yaml.YAMLError as exc:
        raise ValueError(f"Error loading yaml config {p}: {exc}") from exc
    doc = _interpolate(raw)
    return _merge_single_key_lists(doc) if merge_lists else doc


def get_dataset_base_dir() -> Path:
    load_dotenv()
    return Path(os.environ.get("DATASET_DIR", "./"))


def default_config() -> MainConfig:
    return MainConfig()


def apply_yaml(config: MainConfig, config_path) -> MainConfig:
    """Merge a main YAML file (and the group files it names) into ``config``."""
    config_path = Path(config_path)
    doc = load_yaml_config(config_path)
    for group, value in doc.items():
        if group not in GROUPS:
            raise KeyError(f"{group} is not a defined configuration group (known: {', '.join(GROUPS)})")
        target: BaseConfig = getattr(config, group)
        if isinstance(value, str):
            name = value
            sub_path = config_path.parent / group / f"{name}.yaml"
            if hasattr(target, "name"):
                target.name = name
            else:
                setattr(target, "name", name)
            if not sub_path.exists():
                if name == "dummy":
                    continue
                raise FileNotFoundError(f"Config file not found: {sub_path}")
            value = load_yaml_config(sub_path)
        if value is None:
            continue
        if not isinstance(value, dict):
            raise TypeError(f"group '{group}' must be a mapping or a file name, got {type(value).__name__}")
        target.update(**value)
    config.trainer.config_path = str(config_path)
    return config


# --------------------------------------------------------------------------- CLI flags
def _flag_type(tp):
    origin = typing.get_origin(tp)
    if origin is typing.Union:
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        return _flag_type(args[0]) if args else str
    if origin is typing.Literal:
        return str
    if origin in (list, typing.List):
        return None  # nargs
    if tp is bool:
        return lambda s: str(s).lower() in ("1", "true", "yes")
    if tp in (int, float, str):
        return tp
    return str


def build_arg_parser() -> argparse.ArgumentParser:
    """One ``--<field>`` (and ``--<group>.<field>``) flag per scalar option of every group."""
    ap = argparse.ArgumentParser(description="ironcore_b200 trainer options", allow_abbrev=False)
    ap.add_argument("--config-path", "--config", dest="config_path", default=None)
    ap.add_argument("--local-rank", "--local_rank", dest="cli_local_rank", type=int, default=None)
    seen = {"local_rank", "config_path"}
    proto = MainConfig()
    for group in GROUPS:
        gobj = getattr(proto, group)
        hints = typing.get_type_hints(type(gobj))
        for f in fields(gobj):
            if is_dataclass(getattr(gobj, f.name)):
                continue
            tp = hints[f.name]
            ft = _flag_type(tp)
            names = [f"--{group}.{f.name}"]
            if f.name not in seen:
                names += [f"--{f.name}", f"--{f.name.replace('_', '-')}"]
                seen.add(f.name)
            names = list(dict.fromkeys(names))
            kwargs = dict(dest=f"{group}__{f.name}", default=None, help=f.metadata.get("help", ""))
            if ft is None:
                ap.add_argument(*names, nargs="*", **kwargs)
            else:
                ap.add_argument(*names, type=ft, **kwargs)
    return ap


def apply_cli_overrides(config: MainConfig, ns: argparse.Namespace) -> MainConfig:
    for key, value in vars(ns).items():
        if value is None or "__" not in key:
            continue
        group, name = key.split("__", 1)
        getattr(config, group).update(**{name: value})
    return config


def apply_env_ranks(config: MainConfig) -> MainConfig:
    config.parallel.rank = int(os.environ.get("RANK", "0"))
    config.parallel.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config.parallel.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    return config


def _load_special_tokens(config: MainConfig) -> None:
    """Read ``trainer.special_tokens_config_path`` (JSON or YAML: token attribute -> value, e.g. ``eos_token``,
    ``pad_token``, ``eod_token``, or ``*_token_id`` integers) into ``config.data.special_tokens``; the tokenizer
    applies it. A relative path is looked up under ``model.vocab_name_or_path``, then ``trainer.model_path``, then
    the working directory. (Reference: ironcore/config/__init__.py:492-511, ironcore/tokenizer/tokenizer.py:38-40.)"""
    path = config.trainer.special_tokens_config_path
    if not path or getattr(config.data, "special_tokens", None):
        return
    candidates = [Path(path)]
    if not Path(path).is_absolute():
        for base in (config.model.vocab_name_or_path, config.trainer.model_path):
            if base:
                candidates.insert(len(candidates) - 1, Path(base) / path)
    for cand in candidates:
        if cand.exists():
            setattr(config.data, "special_tokens", load_yaml_config(cand))    # (JSON is a subset of YAML)
            return
    raise FileNotFoundError(f"Could not find special token config file: {candidates[0]}")


def load_trainer_config(argv: Optional[Sequence[str]] = None) -> MainConfig:
    """defaults -> YAML (--config-path) -> flag overrides -> env ranks -> validation."""
    load_dotenv()
    ns = build_arg_parser().parse_args(argv)
    config = default_config()
    if ns.config_path:
        apply_yaml(config, ns.config_path)
    apply_cli_overrides(config, ns)
    apply_env_ranks(config)
    if ns.cli_local_rank is not None:
        config.parallel.local_rank = ns.cli_local_rank
    validate_config(config)
    return config


def load_config(config_path, overrides: Optional[Dict[str, Dict[str, Any]]] = None, validate: bool = True) -> MainConfig:
    """Programmatic loader: YAML file plus nested ``{group: {field: value}}`` overrides."""
    load_dotenv()
    config = default_config()
    if config_path is not None:
        apply_yaml(config, config_path)
    for group, kv in (overrides or {}).items():
        getattr(config, group).update(**kv)
    apply_env_ranks(config)
    if validate:
        validate_config(config)
    return config


# --------------------------------------------------------------------------- validation
def data_parallel_size(config: MainConfig) -> int:
    mp = config.trainer.tensor_model_parallel_size * config.trainer.pipeline_model_parallel_size
    if config.parallel.world_size % mp != 0 or config.parallel.world_size < mp:
        raise ValueError(
            f"World size ({config.parallel.world_size}) is not a positive multiple of the model-parallel size ({mp})")
    return config.parallel.world_size // mp


def validate_config(config: MainConfig) -> MainConfig:
    """Check consistency and derive the missing one of {micro batch, global batch, grad-accum}."""
    import torch

    t, m, o, p = config.trainer, config.model, config.operation, config.parallel
    if o.train_steps <= 0:
        raise ValueError("operation.train_steps should be larger than 0")
    if t.pipeline_model_parallel_size != 1:
        raise ValueError("pipeline parallelism is not implemented; pipeline_model_parallel_size must be 1")
    dp = data_parallel_size(config)

    trio = [t.micro_batch_size, t.train_batch_size, t.gradient_accumulation_steps]
    missing = trio.count(None)
    if missing > 1:
        raise ValueError("micro_batch_size, train_batch_size, gradient_accumulation_steps are not sufficiently specified")
    if missing == 1:
        if t.train_batch_size is None:
            t.train_batch_size = t.micro_batch_size * t.gradient_accumulation_steps * dp
        elif t.gradient_accumulation_steps is None:
            t.gradient_accumulation_steps = t.train_batch_size // t.micro_batch_size // dp
        else:
            t.micro_batch_size = t.train_batch_size // t.gradient_accumulation_steps // dp
    if t.micro_batch_size * t.gradient_accumulation_steps * dp != t.train_batch_size:
        raise ValueError(
            "micro_batch_size * gradient_accumulation_steps * data-parallel size should be equal to train_batch_size "
            f"({t.micro_batch_size} * {t.gradient_accumulation_steps} * {dp} != {t.train_batch_size})")

    name = (m.name or "").lower()
    if m.num_attention_groups is None:
        m.num_attention_groups = m.num_attention_heads
    if m.head_dim is None and m.num_attention_heads:
        m.head_dim = m.d_model // m.num_attention_heads
    tp = t.tensor_model_parallel_size
    if tp > 1 and name != "dummy":
        if m.num_attention_heads % tp != 0:
            raise ValueError("num_attention_heads should be divisible by tensor_model_parallel_size")
        if m.num_attention_groups % tp != 0:
            raise ValueError("num_attention_groups should be divisible by tensor_model_parallel_size")
    if name != "dummy" and m.num_attention_heads % m.num_attention_groups != 0:
        raise ValueError("num_attention_heads should be a multiple of num_attention_groups")
    if m.positional_embedding.type.lower() not in ("absolute", "rope", "sinusoidal", "none"):
        raise ValueError("Available positional embedding options are ['absolute', 'rope', 'sinusoidal', 'none'].")
    if p.sequence_parallel and tp > 1 and (t.micro_batch_size * m.max_seq_len) % tp != 0:
        raise ValueError("sequence parallelism needs micro_batch_size * max_seq_len divisible by the TP size")
    ep = p.expert_model_parallel_size
    if ep > 1:
        if m.moe.num_experts <= 0 or m.moe.num_experts % ep != 0:
            raise ValueError("num_experts should be divisible by expert_model_parallel_size")
        if dp % ep != 0:
            raise ValueError("expert_model_parallel_size must divide the data-parallel size")
    if ep > 1 and p.use_fsdp:
        # the shard group of an FSDP unit is the data-parallel group, whose ranks hold *different* experts
        raise ValueError("parallel.use_fsdp with expert_model_parallel_size > 1 is not implemented: shard the "
                         "optimizer state of an expert-parallel model with parallel.zero_stage: 1 instead")
    if p.zero_stage not in (0, 1):
        raise ValueError("zero_stage must be 0 or 1 (use parallel.use_fsdp for full sharding)")
    if config.optim.optimizer.lower() not in ("adam", "adamw", "muon"):
        raise ValueError(f"unknown optimizer {config.optim.optimizer}")
    if not torch.cuda.is_available() and p.dist_backend == "nccl":
        p.dist_backend = "gloo"
    _load_special_tokens(config)
    import warnings

    if m.fp32_residual_connection:
        warnings.warn("model.fp32_residual_connection has no effect: the residual stream stays in the parameter "
                      "dtype (residual adds run in fp32 inside the GEMM and norm kernels)", stacklevel=2)
    if t.compile_model:
        warnings.warn("trainer.compile_model has no effect: the training step launches hand-written kernels; "
                      "trainer.cuda_graph removes the launch overhead that torch.compile would", stacklevel=2)
    return config
