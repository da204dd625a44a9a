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


def _layer_config(heads=4, groups=2, flash=False, rope=False):
    from ironcore.config import (DataConfig, InitConfig, MainConfig, ModelConfig, OperationConfig, OptimConfig,
                                 ParallelConfig, TrainerConfig, UtilsConfig)

    model = ModelConfig(d_model=64, num_attention_heads=heads, num_attention_groups=groups, head_dim=16, max_seq_len=32,
                        max_position_embeddings=32, dropout_attn=0.0, dropout_mlp=0.0, dropout_embd=0.0, no_bias=False,
                        num_layers=2, d_ffn=128)
    if rope:
        model.positional_embedding.type = "rope"
    return MainConfig(model=model, trainer=TrainerConfig(tensor_model_parallel_size=1, use_flash_attn=flash),
                      init=InitConfig(seed=5, init_std=0.02), optim=OptimConfig(max_lr=1e-3), data=DataConfig(),
                      parallel=ParallelConfig(), operation=OperationConfig(train_steps=1), utils=UtilsConfig())


def test_layer_level_call_conventions(compat_path):
    """The reference's layer classes: built from the configuration, ``[b, s, ...]`` tensors in and out."""
    from ironcore.layers import MLP, LanguageModelEmbedding, get_norm
    from ironcore.layers.attention import Attention
    from ironcore.layers.positional_embedding import PositionalEncoding, RotaryPositionalEmbedding
    from ironcore.models.transformer import TransformerLayer, TransformerModel
    from ironcore.parallel import parallel_states
    from ironcore.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    parallel_states.initialize_model_parallel(tensor_model_parallel_size=1, timeout_in_minutes=1.0)
    cfg = _layer_config()
    torch.manual_seed(0)
    b, s, hq, hkv, hd = 2, 12, 4, 2, 16
    q, k, v = torch.randn(b, s, hq, hd), torch.randn(b, s, hkv, hd), torch.randn(b, s, hkv, hd)
    mask = torch.tril(torch.ones(s, s)).expand(b, 1, s, s)
    att = Attention(cfg)
    assert att.num_attention_heads == 4 and att.head_dimension == 16

    def oracle(masked):
        kk, vv = k.repeat_interleave(hq // hkv, 2), v.repeat_interleave(hq // hkv, 2)
        sc = torch.einsum("bqhd,bkhd->bhqk", q, kk) / hd ** 0.5
        if masked:
            sc = sc.masked_fill(mask == 0, float("-inf"))
        return torch.einsum("bhqk,bkhd->bqhd", sc.softmax(-1), vv).reshape(b, s, hq * hd)

    assert torch.allclose(att(q, k, v, mask), oracle(True), atol=1e-5)
    assert torch.allclose(att(q, k, v, attention_mask=None), oracle(False), atol=1e-5)   # no mask: bidirectional

    x = torch.randn(b, s, 64, requires_grad=True)
    layer = TransformerLayer(cfg)
    layer.init_weights()
    assert layer.self_attention is layer.attention
    assert layer.linear_q.weight.shape == (64, 64) and layer.linear_kv.weight.shape == (64, 2 * hkv * hd)
    y = layer(x, mask, rotary_pos_emb=None)
    assert y.shape == x.shape
    y.sum().backward()
    assert x.grad is not None and all(p.grad is not None for p in layer.parameters())
    rope = RotaryPositionalEmbedding(head_dim=hd, max_seq_len=32)
    y_rope = layer(x, mask, rotary_pos_emb=rope)
    assert y_rope.shape == x.shape and not torch.allclose(y_rope, y)
    assert torch.allclose(layer(x, mask, None), y)   # the rotary module of one call does not stick to the layer
    stack = TransformerModel(cfg)
    stack.init_weights()
    assert stack(x, mask, None).shape == x.shape and len(stack.layers) == 2

    col, row = ColumnParallelLinear(cfg, 64, 96, bias=True, concatenated_weights=2), RowParallelLinear(cfg, 96, 64)
    torch.nn.init.normal_(col.weight, std=0.1)
    torch.nn.init.normal_(row.weight, std=0.1)
    h = col(x)
    assert h.shape == (b, s, 96) and torch.allclose(h, x @ col.weight + col.bias, atol=1e-5)
    assert row(h).shape == (b, s, 64)
    mlp = MLP(cfg)
    assert mlp(x).shape == x.shape
    assert get_norm(cfg)(x).shape == x.shape
    emb = LanguageModelEmbedding(cfg)
    ids = torch.randint(0, 100, (b, s))
    assert emb(ids, torch.arange(s).expand(b, s)).shape == (b, s, 64)
    pe = PositionalEncoding(64, max_len=32)
    assert torch.allclose(pe(torch.zeros(b, s, 64))[0], pe(torch.zeros(1, s, 64))[0])
    parallel_states.destroy_model_parallel()


def test_weight_mapper_reference_dialect(compat_path):
    """``WeightMapper(architecture, num_layers)``: the reference's mapper names and ``[out, in]`` weights, and the
    conversion to the live parameter names."""
    from ironcore.checkpointing import Architecture, WeightMapper
    from ironcore.checkpointing.weight_mapping import from_live, to_live

    torch.manual_seed(1)
    d, f, L = 16, 64, 2
    hf = {"transformer.wte.weight": torch.randn(50, d), "transformer.wpe.weight": torch.randn(8, d),
          "transformer.ln_f.weight": torch.randn(d), "transformer.ln_f.bias": torch.randn(d)}
    for i in range(L):
        p = f"transformer.h.{i}."
        hf.update({p + "ln_1.weight": torch.randn(d), p + "ln_1.bias": torch.randn(d), p + "ln_2.weight": torch.randn(d),
                   p + "ln_2.bias": torch.randn(d), p + "attn.c_attn.weight": torch.randn(d, 3 * d),
                   p + "attn.c_attn.bias": torch.randn(3 * d), p + "attn.c_proj.weight": torch.randn(d, d),
                   p + "attn.c_proj.bias": torch.randn(d), p + "mlp.c_fc.weight": torch.randn(d, f),
                   p + "mlp.c_fc.bias": torch.randn(f), p + "mlp.c_proj.weight": torch.randn(f, d),
                   p + "mlp.c_proj.bias": torch.randn(d)})
    mapper = WeightMapper(Architecture.GPT2, num_layers=L)
    ic = mapper.hf_to_ironcore(hf, strict=False)
    assert ic["model.layers.0.self_attention.linear_q.weight"].shape == (d, d)
    assert ic["model.layers.1.self_attention.linear_kv.weight"].shape == (2 * d, d)
    assert ic["model.layers.0.mlp.up_proj.weight"].shape == (f, d) and "output_layernorm.weight" in ic
    back = mapper.ironcore_to_hf(ic, strict=False)
    for k, v in hf.items():
        assert torch.equal(back[k], v), k
    live = to_live(ic)
    assert live["model.layers.0.linear_q.weight"].shape == (d, d) and "output_layernorm.layernorm.weight" in live
    assert live["model.layers.0.mlp.up_proj.weight"].shape == (d, f)
    again = from_live(live)
    assert set(again) == set(ic) and all(torch.equal(again[k], ic[k]) for k in ic)
    assert torch.equal(mapper.ironcore_to_hf(live)["transformer.h.1.attn.c_attn.weight"],
                       hf["transformer.h.1.attn.c_attn.weight"])


def test_reference_signatures_of_helpers(compat_path, tmp_path):
    """Constructors and helpers under the reference's signatures: loggers, timers, tokenizer wrapper, schedules,
    gradient clipping, configuration module paths."""
    import logging

    from ironcore.config.config_trainer import InitConfig, OperationConfig, TrainerConfig  # noqa: F401
    from ironcore.config.config_model import ModelConfig, PositionalEmbeddingConfig  # noqa: F401
    from ironcore.config import print_args
    from ironcore.logger import IronCoreLogger, LevelFormatter, TensorboardLogger
    from ironcore.optimizer.lr_scheduler import CosineAnnealingLR
    from ironcore.optimizer.optimizer import AdamWOptimizer
    from ironcore.tokenizer.tokenizer import Tokenizer
    from ironcore.utils import Timer, bytes_to_mib, clip_grad_norm_tp, get_memory_usage, profile_context

    cfg = _layer_config()
    cfg.utils.tensorboard_dir = str(tmp_path / "tb")
    cfg.trainer.model_name = "m"
    cfg.parallel.rank = 0
    print_args(cfg)
    log = IronCoreLogger(config=cfg, name="compat-test", level=logging.WARNING)
    log.set_log_level(logging.INFO)
    log.info("plain %s", "message")
    log.log_metrics({"hellaswag": {"accuracy": 25.0, "samples": 4}}, msg="evaluation score")
    assert LevelFormatter("%(message)s", level_formats={logging.ERROR: "E %(message)s"}).format(
        logging.LogRecord("x", logging.ERROR, "f", 1, "boom", None, None)) == "E boom"
    tb = TensorboardLogger(cfg)
    tb.add_scalar("loss", 1.0, 0)
    tb.close()
    assert (tmp_path / "tb" / "m").is_dir()

    t = Timer()
    t.register("a")
    with pytest.raises(KeyError):
        t.register("a")
    t.start("a")
    assert t.get("a") >= 0.0 and "a" in t.get_summary()
    t.start("a")
    t.stop_all()
    t.reset_all()
    assert t.get_summary() == {} and bytes_to_mib(3 << 20) == 3 and isinstance(get_memory_usage(in_mib=True), dict)
    with profile_context("tag"):
        pass

    class _Backend:                                  # the surface of a HuggingFace tokenizer that the wrapper reads
        eos_token, eos_token_id, pad_token, pad_token_id, vocab_size = "<eos>", 9, None, None, 10

        def __len__(self):
            return 12

        def encode(self, text):
            return [1, 2]

        def decode(self, ids):
            return "ab"

        def __call__(self, text):
            return {"input_ids": self.encode(text)}

    tok = Tokenizer(_Backend(), "somewhere", vocab_padding_unit=8)
    assert (tok.vocab_size, tok.padded_vocab_size, tok.eos_token_id, tok.eod_token_id, tok.pad_token_id) == (12, 16, 9, 9, 9)
    assert tok("x")["input_ids"] == [1, 2] and tok.decode([1, 2]) == "ab" and tok.decode([]) == "" and tok.pad_token == "<eos>"

    p = torch.nn.Parameter(torch.ones(4))
    opt = AdamWOptimizer([p], lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False)
    sched = CosineAnnealingLR(opt, 2, 4, 10, max_lr=1.0, min_lr=0.1)
    assert opt.param_groups[0]["lr"] == pytest.approx(0.5)
    sched.step()
    assert opt.param_groups[0]["lr"] == pytest.approx(1.0)
    p.grad = torch.full((4,), 3.0)
    norm = clip_grad_norm_tp([p], max_norm=3.0)
    assert norm.item() == pytest.approx(6.0) and p.grad.norm().item() == pytest.approx(3.0, rel=1e-4)


def test_reference_style_huggingface_directory_round_trip(compat_path, tmp_path):
    """``load_from_huggingface(path, model)`` / ``export_to_huggingface(model, path, architecture=...)`` on a
    directory written by ``transformers``: same logits, same tensors back."""
    transformers = pytest.importorskip("transformers")
    from ironcore.checkpointing import export_to_huggingface, load_from_huggingface
    from ironcore.checkpointing.hf_interop import detect_checkpoint_format, load_hf_config, load_hf_state_dict
    from ironcore_b200.config import validate_config
    from ironcore_b200.models.language_model import LanguageModel
    from ironcore_b200.parallel import mesh
    from helpers import tiny_config

    hcfg = transformers.LlamaConfig(vocab_size=96, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                    rms_norm_eps=1e-5, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(hcfg).eval()
    src = tmp_path / "hf_in"
    hf.save_pretrained(src, safe_serialization=True)
    assert load_hf_config(src)["model_type"] == "llama" and detect_checkpoint_format(src)
    assert "model.embed_tokens.weight" in load_hf_state_dict(src, device="cpu")

    mesh.destroy_model_parallel()
    cfg = tiny_config("llama", d_model=32, d_ffn=64, num_attention_heads=4, num_attention_groups=2, head_dim=8,
                      vocab_size=96, ln_eps=1e-5, hf_model_type="llama")
    cfg.data.vocab_size = 96
    validate_config(cfg)
    model = LanguageModel(cfg).eval()
    info = load_from_huggingface(src, model)
    assert info["missing_keys"] == [] and "embedding.word_embeddings.weight" in info["loaded_keys"]
    ids = torch.randint(0, 96, (2, 16))
    with torch.no_grad():
        assert torch.allclose(model(ids)[..., :96], hf(ids).logits, atol=2e-4)
    out = export_to_huggingface(model, tmp_path / "hf_out", architecture="llama")
    assert out["config_file"] and out["files"]
    back = load_hf_state_dict(tmp_path / "hf_out")
    for k, v in hf.state_dict().items():
        assert torch.allclose(back[k], v, atol=1e-6), k


def test_reference_helper_methods_of_the_language_model(compat_path):
    from ironcore_b200.config import validate_config
    from ironcore_b200.models.language_model import LanguageModel
    from ironcore_b200.parallel import mesh
    from helpers import tiny_config

    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2")
    cfg.model(reset_position_ids=True, reset_attention_mask=True, eod_mask_loss=True, eod_token_id=7, pad_token_id=0)
    validate_config(cfg)
    model = LanguageModel(cfg).eval()
    ids = torch.tensor([[3, 4, 7, 5, 6, 7, 8, 9]])
    labels = torch.tensor([[4, 7, 5, 6, 7, 8, 9, 0]])
    mask, pos, lmask = model.get_masks_and_position_ids(ids, labels)
    assert pos.tolist() == [[0, 1, 2, 0, 1, 2, 0, 1]]
    assert mask.shape == (1, 1, 8, 8) and bool(mask[0, 0, 4, 3]) and not bool(mask[0, 0, 3, 2]) and not bool(mask[0, 0, 1, 2])
    assert lmask.tolist() == [[1, 0, 1, 1, 0, 1, 1, 0]]
    with torch.no_grad():
        logits = model(ids)
        loss = model(ids, labels)
        again = model.compute_loss_from_logits(logits, labels, lmask)
        hidden, _ = model.hidden_states(ids)
        assert torch.allclose(model.post_lm_processing(hidden.view(1, 8, -1)), logits, atol=1e-5)
        assert torch.allclose(model.post_lm_processing(hidden.view(1, 8, -1), labels, lmask), again, atol=1e-6)
    assert loss.item() == pytest.approx(again.item(), rel=1e-5)


def test_reference_data_constructors(compat_path, tmp_path):
    import numpy as np

    from ironcore.dataloader import BinaryDataset, DataConfig, WeightedMixingDataset, create_collator, load_data_config
    from ironcore_b200.data.serializer import BIN_NAME, IDX_DTYPE, IDX_NAME

    d = tmp_path / "pre" / "toy" / "pretrain"
    d.mkdir(parents=True)
    toks = (np.arange(400) % 50).astype(np.uint16)
    toks.tofile(d / BIN_NAME)
    idx = np.zeros(4, dtype=IDX_DTYPE)
    idx["offset"], idx["length"], idx["type"] = [0, 100, 200, 300], 100, "pretrain"
    np.save(d / IDX_NAME, idx)
    y = tmp_path / "data.yaml"
    y.write_text(f"train_datasets:\n  - name: toy\n    source: none\n    task_type: pretrain\n    ratio: 1.0\n"
                 f"seq_length: 16\nsplits: [1.0, 0.0, 0.0]\npreprocessed_dir: {tmp_path / 'pre'}\n")
    dcfg = load_data_config(y)
    assert isinstance(dcfg, DataConfig) and dcfg.get_dataset_output_path(dcfg.datasets[0]) == d
    ds = BinaryDataset(d / BIN_NAME, d / IDX_NAME)
    assert ds.total_tokens() == 400 and len(ds) == 4 and len(ds[1]["token_ids"]) == 100
    mix = WeightedMixingDataset(dcfg, mode="pretrain", seed=1, split="train")
    first = next(iter(mix))
    assert len(first["tokens"]) == 17
    coll = create_collator("sft", 8, pad_token_id=0, return_full_attention_mask=True, use_flash_attention=False)
    batch = coll([{"tokens": np.arange(1, 6), "mask_ranges": [[0, 2]]}, {"tokens": np.arange(1, 4), "mask_ranges": []}])
    m = batch["attention_mask"]
    assert "cu_seqlens" not in batch and m.shape == (1, 8, 8) and bool(m[0, 4, 0]) and not bool(m[0, 5, 4]) and bool(m[0, 6, 5])
