"""Data side-chain: serialisation format round trip, integrity checks, datasets, collators."""

import json

import numpy as np
import pytest
import torch
import yaml


def _write_sources(tmp_path):
    pre = tmp_path / "pre.jsonl"
    with open(pre, "w") as f:
        for i in range(40):
            f.write(json.dumps({"text": f"document number {i} " + "lorem ipsum " * (5 + i % 7)}) + "\n")
    sft = tmp_path / "sft.jsonl"
    with open(sft, "w") as f:
        for i in range(12):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"question {i}?"},
                                             {"role": "assistant", "content": f"answer {i} " * (1 + i % 4)}]}) + "\n")
    dpo = tmp_path / "dpo.jsonl"
    with open(dpo, "w") as f:
        for i in range(6):
            f.write(json.dumps({"prompt": f"p{i}", "chosen": f"good {i}", "rejected": f"bad {i}"}) + "\n")
    cfg = {"tokenizer_type": "bbpe", "vocab_name_or_path": "none", "seq_length": 64, "splits": [0.8, 0.2, 0.0],
           "preprocessed_dir": str(tmp_path / "out"),
           "train_datasets": [{"name": "pre", "dataset_path": str(pre), "task_type": "pretrain", "ratio": 1.0},
                              {"name": "chat", "dataset_path": str(sft), "task_type": "sft", "ratio": 1.0},
                              {"name": "pref", "dataset_path": str(dpo), "task_type": "dpo", "ratio": 1.0}]}
    p = tmp_path / "data.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return p


def test_preprocess_inspect_and_load(tmp_path, capsys):
    from ironcore_b200.__main__ import main
    from ironcore_b200.cli.inspect import check_integrity, statistics
    from ironcore_b200.data.collator import UniversalCollator
    from ironcore_b200.data.data_config import UniversalDataConfig
    from ironcore_b200.data.dataset import BinaryDataset, WeightedMixingDataset

    cfg_path = _write_sources(tmp_path)
    assert main(["preprocess", "--config", str(cfg_path), "--inspect", "--preview", "1"]) == 0
    dcfg = UniversalDataConfig.from_yaml(cfg_path)
    pre_dir = dcfg.datasets[0].output_path
    assert check_integrity(pre_dir) == []
    st = statistics(pre_dir)
    assert st["samples"] == 40 and st["types"] == {"pretrain": 40}
    ds = BinaryDataset(pre_dir)
    assert ds.tokens.dtype == np.uint16
    rec = ds.sample(3)
    assert rec["tokens"][-1] == 50256  # EOS appended
    # pretrain windows: two ranks see disjoint positions
    mk = lambda r: WeightedMixingDataset([pre_dir], [1.0], "pretrain", "train", 16, dcfg.splits, dp_rank=r, dp_size=2,
                                         epochs=1)
    a = [tuple(x["tokens"].tolist()) for x in mk(0)]
    b = [tuple(x["tokens"].tolist()) for x in mk(1)]
    assert a and b and all(len(t) == 17 for t in a)
    batch = UniversalCollator("pretrain", 16)([{"tokens": np.asarray(a[0])}, {"tokens": np.asarray(a[1])}])
    assert batch["input_ids"].shape == (2, 16) and torch.equal(batch["input_ids"][:, 1:], batch["labels"][:, :-1])
    # corrupt the index: integrity check must notice
    idx = np.load(pre_dir / "data.idx.npy")
    idx["offset"][5] += 3
    np.save(pre_dir / "data.idx.npy", idx)
    assert check_integrity(pre_dir)


def test_sft_packing_and_masks(tmp_path):
    from ironcore_b200.__main__ import main
    from ironcore_b200.data.collator import IGNORE_INDEX, UniversalCollator, first_fit_decreasing
    from ironcore_b200.data.data_config import UniversalDataConfig
    from ironcore_b200.data.dataset import WeightedMixingDataset

    assert first_fit_decreasing([5, 4, 3, 2], 6) == [[0], [1, 3], [2]]
    cfg_path = _write_sources(tmp_path)
    assert main(["preprocess", "--config", str(cfg_path)]) == 0
    dcfg = UniversalDataConfig.from_yaml(cfg_path)
    sft_dir = dcfg.datasets[1].output_path
    ds = WeightedMixingDataset([sft_dir], [1.0], "sft", "train", 64, [1.0, 0.0, 0.0], epochs=1)
    samples = list(ds)
    assert len(samples) == 12 and all(s["mask_ranges"] for s in samples)
    batch = UniversalCollator("sft", 64, pad_token_id=0)(samples)
    ids, labels, pos, cu = batch["input_ids"], batch["labels"], batch["position_ids"], batch["cu_seqlens"]
    assert ids.shape == labels.shape == pos.shape and ids.shape[1] == 64
    assert int(cu[0]) == 0 and int(cu[-1]) == ids.numel()
    assert (labels != IGNORE_INDEX).any() and (labels == IGNORE_INDEX).any()
    # positions restart at every packed sample
    assert int((pos == 0).sum()) >= len(samples)
    dpo_dir = dcfg.datasets[2].output_path
    pairs = list(WeightedMixingDataset([dpo_dir], [1.0], "dpo", "train", 64, [1.0, 0.0, 0.0], epochs=1))
    assert len(pairs) == 6
    b = UniversalCollator("dpo", 64)(pairs)
    assert "chosen_input_ids" in b and "rejected_labels" in b


def test_trainer_on_preprocessed_files(tmp_path):
    from helpers import tiny_config
    from ironcore_b200.__main__ import main
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    cfg_path = _write_sources(tmp_path)
    assert main(["preprocess", "--config", str(cfg_path)]) == 0
    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2", vocab_size=50257)
    cfg.data(task_type="pretrain", config_path=str(cfg_path), vocab_size=50257)
    cfg.operation.train_steps = 2
    validate_config(cfg)
    tr = Trainer(cfg)
    losses = [float(tr.train_step(s)[0]) for s in range(2)]
    assert all(np.isfinite(losses))


def test_long_conversation_masks_survive_serialisation(tmp_path):
    """A 70-turn conversation has more mask ranges than the 500-character index field holds: they go to
    the side table, every user turn stays masked, and the record reads back identical."""
    from ironcore_b200.data.data_config import DatasetConfig, UniversalDataConfig
    from ironcore_b200.data.dataset import BinaryDataset
    from ironcore_b200.data.serializer import RANGES_NAME, DataSerializer
    from ironcore_b200.tokenizer import Tokenizer

    msgs = []
    for i in range(70):
        msgs.append({"role": "user", "content": f"question number {i} with some padding text"})
        msgs.append({"role": "assistant", "content": f"reply {i}"})
    short = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]
    src = tmp_path / "long.jsonl"
    src.write_text(json.dumps({"messages": msgs}) + "\n" + json.dumps({"messages": short}) + "\n")
    ds_cfg = DatasetConfig(name="long", source=str(src), task_type="sft", output_path=tmp_path / "out")
    tok = Tokenizer(50257, 50256, None)
    ser = DataSerializer(UniversalDataConfig(datasets=[ds_cfg]), tok)
    want_tokens, want_masks = ser._chat_tokens(msgs)
    assert len(want_masks) == 70 and len(json.dumps(want_masks)) > 500
    ser.serialize(ds_cfg, force=True)
    assert (tmp_path / "out" / RANGES_NAME).exists()
    ds = BinaryDataset(tmp_path / "out")
    rec = ds.sample(0)
    assert rec["mask_ranges"] == want_masks and rec["tokens"].tolist() == want_tokens
    assert str(ds.index[0]["mask_ranges"]).startswith("@")
    assert ds.sample(1)["mask_ranges"] == ser._chat_tokens(short)[1]      # short ones stay inline JSON
    assert str(ds.index[1]["mask_ranges"]).startswith("[")


def test_chat_template_of_the_tokenizer_is_used(tmp_path):
    """With a tokenizer that carries a chat template the serializer renders through it and masks the
    non-assistant turns by prefix rendering."""
    from ironcore_b200.data.data_config import DatasetConfig, UniversalDataConfig
    from ironcore_b200.data.serializer import DataSerializer

    class TemplateTok:
        eos_token_id = 1
        vocab_size = 300
        chat_template = "stub"

        def encode(self, text):
            return [ord(c) % 256 for c in text]

        def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=False, chat_template=None):
            tag = chat_template or self.chat_template
            text = "<bos>" + "".join(f"[{tag}:{m['role']}]{m['content']}</s>" for m in messages)
            return self.encode(text)

    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "2+2?"},
            {"role": "assistant", "content": "4"}, {"role": "user", "content": "3+3?"},
            {"role": "assistant", "content": "6"}]
    dummy = DatasetConfig(name="d", source=str(tmp_path), task_type="sft")
    ser = DataSerializer(UniversalDataConfig(datasets=[dummy]), TemplateTok())
    tokens, masks = ser._chat_tokens(msgs)
    text = "".join(chr(t) for t in tokens)
    assert text.startswith("<bos>[stub:system]")
    kept = "".join(c for i, c in enumerate(text) if not any(a <= i < b for a, b in masks))
    assert kept == "[stub:assistant]4</s>[stub:assistant]6</s>"
    # a per-dataset template overrides the tokenizer's
    tokens2, _ = ser._chat_tokens(msgs, template="custom")
    assert "[custom:user]" in "".join(chr(t) for t in tokens2)


def test_pretrain_mixing_follows_the_ratios(tmp_path):
    from ironcore_b200.data.dataset import WeightedMixingDataset
    from ironcore_b200.data.serializer import BIN_NAME, IDX_DTYPE, IDX_NAME

    dirs = []
    for name, fill in (("a", 7), ("b", 9)):
        d = tmp_path / name
        d.mkdir()
        np.full(16 * 400, fill, dtype=np.uint16).tofile(d / BIN_NAME)
        np.save(d / IDX_NAME, np.array([(0, 16 * 400, "pretrain", 0, "[]")], dtype=IDX_DTYPE))
        dirs.append(d)
    ds = WeightedMixingDataset(dirs, [0.9, 0.1], "pretrain", "train", 16, [1.0, 0.0, 0.0], epochs=1)
    firsts = [int(x["tokens"][0]) for x in ds]
    assert len(firsts) == 800
    share_a = firsts.count(7) / len(firsts)
    assert abs(share_a - 0.9) < 0.01, share_a
    # both ranks together see the same multiset, split evenly
    r0 = list(WeightedMixingDataset(dirs, [0.9, 0.1], "pretrain", "train", 16, [1.0, 0.0, 0.0], dp_rank=0, dp_size=2, epochs=1))
    r1 = list(WeightedMixingDataset(dirs, [0.9, 0.1], "pretrain", "train", 16, [1.0, 0.0, 0.0], dp_rank=1, dp_size=2, epochs=1))
    assert len(r0) + len(r1) == 800 and abs(len(r0) - len(r1)) <= 1


def test_preference_pairs_from_files_train_with_dpo(tmp_path, capsys):
    """``ironcore preprocess`` on a file of (prompt, chosen, rejected) rows, then ``ironcore train`` with
    ``data.task_type: dpo``: the command-line path picks the DPO trainer and runs its steps."""
    from ironcore_b200.__main__ import main
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg_path = _write_sources(tmp_path)
    assert main(["preprocess", "--config", str(cfg_path)]) == 0
    run = {"trainer": {"micro_batch_size": 2, "train_batch_size": 2, "log_interval": 1, "model_path": "",
                       "use_flash_attn": False, "vocab_padding_unit": 8},
           "operation": {"train_steps": 3, "no_save": True},
           "model": {"name": "gpt2", "d_model": 32, "d_ffn": 64, "num_layers": 2, "num_attention_heads": 4,
                     "max_seq_len": 64, "max_position_embeddings": 64, "precision": "fp32", "dropout_embd": 0.0,
                     "dropout_attn": 0.0, "dropout_mlp": 0.0},
           "data": {"task_type": "dpo", "config_path": str(cfg_path)},
           "optim": {"max_lr": 1e-3, "warmup_steps": 0}, "rl": {"dpo_beta": 0.2}}
    run_path = tmp_path / "run.yaml"
    run_path.write_text(yaml.safe_dump(run))
    assert main(["train", "--config", str(run_path)]) == 0
    out = capsys.readouterr().out
    assert "Task type: dpo" in out and "Training completed successfully" in out
    mesh.destroy_model_parallel()


@pytest.mark.parametrize("task", ["pretrain", "sft", "dpo"])
def test_file_backed_stream_can_start_further_in(tmp_path, task):
    """``skip_batches`` before the first batch moves the dataset's starting point (no tokens are read for the part
    passed over); the batches that follow are the ones an iterator that drew and dropped would have produced."""
    from helpers import tiny_config
    from ironcore_b200.__main__ import main
    from ironcore_b200.config import validate_config
    from ironcore_b200.data import get_data_iterator

    cfg_path = _write_sources(tmp_path)
    assert main(["preprocess", "--config", str(cfg_path)]) == 0

    def stream():
        cfg = tiny_config("gpt2", vocab_size=50257)
        cfg.data(task_type=task, config_path=str(cfg_path), vocab_size=50257)
        cfg.trainer(micro_batch_size=2, train_batch_size=2, gradient_accumulation_steps=None)
        validate_config(cfg)
        return get_data_iterator(cfg, dp_rank=0, dp_size=1)["train"]

    plain, moved = stream(), stream()
    for _ in range(2):
        next(plain)
    moved.skip_batches(2)
    for _ in range(2):
        a, b = next(plain), next(moved)
        assert a.keys() == b.keys()
        for k in a:
            assert torch.equal(a[k], b[k]), k
    moved.skip_batches(1)                 # after the first draw: batches are drawn and dropped
    next(plain)
    a, b = next(plain), next(moved)
    assert all(torch.equal(a[k], b[k]) for k in a)
