"""Every YAML preset under configs/ loads and validates; every model preset builds (shrunk) and runs."""

from __future__ import annotations

import glob
import os

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNS = sorted(p for p in glob.glob(os.path.join(ROOT, "configs", "*.yaml")))
MODELS = sorted(glob.glob(os.path.join(ROOT, "configs", "model", "*.yaml")))
DATA = sorted(glob.glob(os.path.join(ROOT, "configs", "data", "*.yaml")))


@pytest.mark.parametrize("path", RUNS, ids=[os.path.basename(p) for p in RUNS])
def test_run_preset_loads(path, monkeypatch):
    from ironcore_b200.config import load_config

    world = {"baseline_llama7b_tp8.yaml": 8, "baseline_moe_ep8.yaml": 8, "baseline_llama13b_fsdp_muon.yaml": 8,
             "baseline_grpo_qwen.yaml": 8, "example.yaml": 2, "dpo_example.yaml": 2,
             "finetune_from_hf_example.yaml": 8}.get(os.path.basename(path), 1)
    monkeypatch.setenv("WORLD_SIZE", str(world))
    monkeypatch.setenv("RANK", "0")
    monkeypatch.chdir(ROOT)
    cfg = load_config(path)
    assert cfg.trainer.gradient_accumulation_steps >= 1
    assert cfg.model.name


def test_baseline_presets_match_the_named_shapes(monkeypatch):
    from ironcore_b200.config import load_config

    monkeypatch.setenv("WORLD_SIZE", "8")
    monkeypatch.setenv("RANK", "0")
    monkeypatch.chdir(ROOT)
    c = load_config("configs/baseline_llama7b_tp8.yaml")
    m = c.model
    assert (m.num_layers, m.d_model, m.num_attention_heads, m.head_dim, m.d_ffn) == (32, 4096, 32, 128, 11008)
    assert c.trainer.tensor_model_parallel_size == 8 and c.parallel.sequence_parallel and c.parallel.zero_stage == 1
    assert c.trainer.train_batch_size == 64 and m.max_seq_len == 4096
    c = load_config("configs/baseline_moe_ep8.yaml")
    assert (c.model.moe.num_experts, c.model.moe.top_k, c.model.moe.num_shared_experts) == (64, 6, 2)
    assert c.parallel.expert_model_parallel_size == 8 and c.model.num_attention_groups == 4
    c = load_config("configs/baseline_llama13b_fsdp_muon.yaml")
    assert c.parallel.use_fsdp and c.optim.optimizer == "muon" and c.optim.cpu_offload_optimizer
    assert (c.model.num_layers, c.model.d_model, c.model.d_ffn) == (40, 5120, 13824)
    c = load_config("configs/baseline_grpo_qwen.yaml")
    assert (c.model.num_layers, c.model.d_model, c.model.num_attention_groups, c.model.d_ffn) == (28, 1536, 2, 8960)
    assert c.model.qkv_bias and c.rl.group_size == 8 and c.rl.kv_block_size == 16 and c.rl.max_new_tokens == 512


@pytest.mark.parametrize("path", MODELS, ids=[os.path.basename(p) for p in MODELS])
def test_model_preset_builds_and_steps(path):
    """The preset's architecture switches, shrunk to a toy size, produce a finite loss and gradients."""
    from ironcore_b200.config import default_config, validate_config
    from ironcore_b200.config.loader import load_yaml_config
    from ironcore_b200.parallel import mesh

    y = load_yaml_config(path)
    heads, groups = int(y["num_attention_heads"]), int(y.get("num_attention_groups") or y["num_attention_heads"])
    g = 1 if groups == 1 else 2
    shrink = dict(num_layers=2, d_model=64, d_ffn=96, num_attention_heads=4, num_attention_groups=g if groups != heads else 4,
                  head_dim=16, max_seq_len=32, max_position_embeddings=32, precision="fp32", vocab_size=256,
                  dropout_embd=0.0, dropout_attn=0.0, dropout_mlp=0.0)
    y.update(shrink)
    if isinstance(y.get("moe"), dict) and y["moe"].get("num_experts"):
        y["moe"].update(num_experts=4, top_k=2, expert_d_ffn=32, shared_expert_d_ffn=32)
    c = default_config()
    c.model(**y)
    c.data(task_type="synthetic", vocab_size=256)
    c.trainer(micro_batch_size=2, train_batch_size=2, vocab_padding_unit=8)
    c.parallel(world_size=1, rank=0)
    validate_config(c)
    mesh.destroy_model_parallel()
    from ironcore_b200.trainer import Trainer

    c.operation(train_steps=2, no_save=True)
    tr = Trainer(c)
    loss, _, _ = tr.train_step(0)
    assert torch.isfinite(loss)
    assert all(torch.isfinite(p).all() for p in tr.model.parameters())


@pytest.mark.parametrize("path", DATA, ids=[os.path.basename(p) for p in DATA])
def test_data_preset_parses(path):
    from ironcore_b200.config.loader import load_yaml_config

    y = load_yaml_config(path, merge_lists=False)
    if os.path.basename(path) == "base.yaml":
        assert "train" in y
        return
    from ironcore_b200.data.data_config import UniversalDataConfig

    cfg = UniversalDataConfig.from_yaml(path) if hasattr(UniversalDataConfig, "from_yaml") else UniversalDataConfig(**y)
    assert cfg.datasets and cfg.seq_length > 0 and abs(sum(d.ratio for d in cfg.datasets) - 1.0) < 1e-6


def test_every_configuration_field_is_documented():
    """configs/README.md lists every field of every configuration group (name in the group's table)."""
    from dataclasses import fields, is_dataclass

    from ironcore_b200.config import default_config

    text = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "README.md")).read()
    sections = {}
    current = None
    for line in text.split("\n"):
        if line.startswith("###"):
            current = line.lstrip("# ").strip()
            sections[current] = []
        elif current is not None and line.startswith("| `"):
            sections[current].append(line.split("`")[1])

    def check(node, title):
        assert title in sections, f"group {title} has no table"
        for f in fields(node):
            assert f.name in sections[title], f"{title}.{f.name} is not documented"
            v = getattr(node, f.name)
            if is_dataclass(v):
                check(v, f"{title}.{f.name}")

    cfg = default_config()
    for f in fields(cfg):
        check(getattr(cfg, f.name), f.name)
