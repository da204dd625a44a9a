"""The ``ironcore`` import package (the reference's public names) and the extra CLI sub-command."""

import importlib
import json
import os
import pkgutil
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture()
def compat_path():
    p = os.path.join(ROOT, "compat")
    sys.path.insert(0, p)
    yield p
    sys.path.remove(p)
    for name in [m for m in sys.modules if m == "ironcore" or m.startswith("ironcore.")]:
        del sys.modules[name]


def test_reference_names_resolve(compat_path):
    import ironcore

    assert os.path.dirname(ironcore.__file__).startswith(compat_path)
    for m in pkgutil.walk_packages(ironcore.__path__, "ironcore."):
        importlib.import_module(m.name)
    from ironcore import get_config, get_logger, get_timer, get_tokenizer, set_global_states  # noqa: F401
    from ironcore.checkpointing import (WeightMapper, export_to_huggingface, load_checkpoint,  # noqa: F401
                                        load_from_huggingface, save_checkpoint)
    from ironcore.config import MainConfig, _config_validation, load_trainer_config  # noqa: F401
    from ironcore.dataloader import get_data_iterator  # noqa: F401
    from ironcore.language_model import LanguageModel  # noqa: F401
    # the submodule paths that the reference's own examples and tests import from
    from ironcore.checkpointing.hf_interop import _generate_hf_config, load_hf_config, load_hf_state_dict  # noqa: F401
    from ironcore.checkpointing.weight_mapping import ARCHITECTURE_ALIASES, get_architecture  # noqa: F401
    from ironcore.eval.tasks.hellaswag import HellaSwag  # noqa: F401
    from ironcore.layers.attention import Attention  # noqa: F401
    from ironcore.layers.positional_embedding.rotary import RotaryPositionalEmbedding  # noqa: F401
    from ironcore.models.transformer import TransformerLayer  # noqa: F401
    from ironcore.preprocessing import DataSerializer  # noqa: F401
    from ironcore.tokenizer.tokenizer import build_tokenizer  # noqa: F401
    from ironcore.utils import get_device, get_model_dtype, is_first_rank, profile_context  # noqa: F401
    from ironcore.training_utils import forward_step, loss_func  # noqa: F401
    assert get_architecture("llama-3").value == "llama" and "gpt2" in ARCHITECTURE_ALIASES
    from ironcore.optimizer import AdamWOptimizer, CosineAnnealingLR, get_lr_scheduler, get_optimizer  # noqa: F401
    from ironcore.parallel import initialize_parallelism, initialize_process  # noqa: F401
    from ironcore.parallel.parallel_states import (get_data_parallel_group, get_data_parallel_group_rank,  # noqa: F401
                                                   get_data_parallel_world_size, get_tensor_model_parallel_group,
                                                   get_tensor_model_parallel_group_rank,
                                                   get_tensor_model_parallel_rank,
                                                   get_tensor_model_parallel_world_size, initialize_model_parallel)
    from ironcore.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear,  # noqa: F401
                                                   VocabParallelEmbedding, copy_inputs_to_model_parallel_workers,
                                                   reduce_inputs_from_model_parallel_workers,
                                                   scatter_input_to_model_parallel_workers,
                                                   vocab_parallel_cross_entropy)
    from ironcore.parallel.tensor_parallel.comm import (gather_from_model_parallel_workers,  # noqa: F401
                                                        split_to_model_parallel_workers)
    from ironcore.trainer import Trainer
    from ironcore.training_utils import forward_step, loss_func  # noqa: F401
    from ironcore_b200.trainer import Trainer as Native

    assert Trainer is Native
    x = torch.randn(3, 4)
    assert copy_inputs_to_model_parallel_workers(x) is x or torch.equal(copy_inputs_to_model_parallel_workers(x), x)
    assert get_tensor_model_parallel_group_rank() == 0 and get_data_parallel_world_size() == 1


def test_reference_style_training_script(compat_path):
    """The way the reference's examples/train.py drives a run: config -> validation -> Trainer(config,
    forward_step, loss_func) -> train_step."""
    from helpers import tiny_config
    from ironcore.config import _config_validation
    from ironcore.trainer import Trainer
    from ironcore.training_utils import forward_step, loss_func
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2")
    _config_validation(cfg)
    with Trainer(cfg, forward_step, loss_func) as tr:
        loss = float(tr.train_step(0)[0])
    assert loss == loss and loss < 20


def test_inspect_subcommand(tmp_path, capsys):
    import yaml

    from ironcore_b200.__main__ import main

    src = tmp_path / "pre.jsonl"
    src.write_text("".join(json.dumps({"text": f"doc {i} " + "abc " * 20}) + "\n" for i in range(10)))
    cfg = {"tokenizer_type": "bbpe", "vocab_name_or_path": "none", "seq_length": 32, "splits": [1.0, 0.0, 0.0],
           "preprocessed_dir": str(tmp_path / "out"),
           "train_datasets": [{"name": "pre", "dataset_path": str(src), "task_type": "pretrain", "ratio": 1.0}]}
    p = tmp_path / "data.yaml"
    p.write_text(yaml.safe_dump(cfg))
    assert main(["preprocess", "--config", str(p)]) == 0
    assert main(["inspect", "--config", str(p), "--preview", "1"]) == 0
    out = capsys.readouterr().out
    assert "[pre]" in out and "OK" in out
    assert (tmp_path / "out" / "inspection_report.json").exists()


def test_reference_style_evaluation_script(compat_path, tmp_path):
    """The way the reference's evaluation / generation scripts set a model up (tests/test_eval.py:28-60,
    examples/generate_text.py): global states, process and model-parallel initialisation, LanguageModel(config),
    initialize_parallelism, load_checkpoint (-1 without a checkpoint), then a forward pass for logits."""
    from helpers import tiny_config
    from ironcore import get_logger, set_global_states
    from ironcore.checkpointing import load_checkpoint
    from ironcore.language_model import LanguageModel
    from ironcore.parallel import initialize_parallelism, initialize_process
    from ironcore.parallel.parallel_states import initialize_model_parallel
    from ironcore.utils import get_device, get_model_dtype, is_first_rank
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = tiny_config("llama")
    cfg.trainer.model_path = str(tmp_path / "ckpt")
    set_global_states(cfg)
    initialize_process(cfg)
    assert get_logger() is not None and is_first_rank()
    device, dtype = get_device(), get_model_dtype(cfg)
    initialize_model_parallel(cfg.trainer.tensor_model_parallel_size, timeout=cfg.parallel.timeout_minute)
    model = LanguageModel(cfg).to(device=device, dtype=dtype)
    model = initialize_parallelism(cfg, model)
    assert load_checkpoint(cfg, model) == -1
    ids = torch.randint(0, cfg.model.vocab_size or cfg.data.vocab_size, (2, 16))
    with torch.no_grad():
        logits = model(ids)
    assert logits.shape[:2] == (2, 16) and torch.isfinite(logits).all()
