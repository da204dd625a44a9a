"""Auxiliary subsystems on CPU: failure detection on the host, cadence control, LR schedule, eval task,
config loading from YAML groups, corrupted checkpoint handling."""

import json
import os

import pytest
import torch
import yaml

from helpers import run_distributed, tiny_config


# ------------------------------------------------------------------ failure detection (host only)
class _FakeStore:
    def __init__(self):
        self.kv = {}

    def set(self, k, v):
        self.kv[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        if k not in self.kv:
            raise AssertionError("a get() of a missing key blocks on a real store")
        return self.kv[k]

    def check(self, keys):
        return all(k in self.kv for k in keys)


def test_heartbeat_detects_silent_rank_with_fake_clock():
    from ironcore_b200.parallel.fault import Heartbeat, RankFailure

    now = [1000.0]
    store = _FakeStore()
    a = Heartbeat(0, 10.0, store, rank=0, world_size=3, clock=lambda: now[0])
    b = Heartbeat(0, 10.0, store, rank=1, world_size=3, clock=lambda: now[0])
    assert a.dead_peers() == []             # rank 2 has not joined yet, but the timeout has not passed either
    now[0] += 11.0
    b.beat(0)
    assert a.dead_peers() == [2]            # ... now it has: a rank that never publishes is reported
    c = Heartbeat(0, 10.0, store, rank=2, world_size=3, clock=lambda: now[0])
    assert a.dead_peers() == []
    now[0] += 8.0
    b.beat(5)
    assert a.dead_peers() == []
    now[0] += 8.0                            # rank 2 silent for 16 s, rank 1 for 8 s
    assert a.dead_peers() == [2]
    assert a.peer_steps() == {1: 5, 2: -1}
    with pytest.raises(RankFailure) as e:
        a.raise_if_peer_dead()
    assert e.value.ranks == [2]
    c.beat(6)
    a.raise_if_peer_dead()


def _hb_worker(rank, world):
    import time

    from ironcore_b200.parallel.fault import Heartbeat

    hb = Heartbeat(interval_s=0.05, timeout_s=0.6)
    if rank == 1:
        hb.stop()               # this rank stops publishing (a hung or dead process), between steps
        time.sleep(1.5)
        return
    time.sleep(1.2)
    dead = hb.dead_peers()
    hb.stop()
    assert dead == [1], dead


def test_heartbeat_over_real_store_two_ranks():
    run_distributed(_hb_worker, 2)


def _leave_worker(rank, world):
    """Three ranks train with heartbeats; after step 0, between steps and with nothing in flight, rank 2 leaves
    (a host-side exception in its loop). The others read its tombstone before their next step and stop with a
    ``RankFailure`` at once, long before the heartbeat timeout, instead of entering a collective."""
    import time

    import torch.distributed as dist

    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel.fault import RankFailure
    from ironcore_b200.trainer import Trainer

    cfg = tiny_config("gpt2")
    cfg.trainer(micro_batch_size=1, train_batch_size=3, gradient_accumulation_steps=None)
    cfg.parallel(world_size=world, rank=rank)
    cfg.utils(heartbeat_interval_s=0.1, heartbeat_timeout_s=120.0)
    validate_config(cfg)
    tr = Trainer(cfg)
    hb = tr.heartbeat
    assert hb is not None
    hb.beat(0)
    hb.raise_if_peer_dead()
    tr.train_step(0)
    if rank == 2:
        hb.leave("injected failure")
    dist.barrier()          # (test only) orders the tombstone before the others' next question
    if rank == 2:
        return
    t0 = time.time()
    with pytest.raises(RankFailure) as info:
        hb.beat(1)
        hb.raise_if_peer_dead()
    assert info.value.ranks == [2] and time.time() - t0 < 5.0
    hb.stop()


def test_rank_that_leaves_between_steps_stops_its_peers():
    run_distributed(_leave_worker, 3)


def _timeout_worker(rank, world):
    """A rank that never joins a collective: the short process-group timeout ends the others' wait
    with an error instead of a hang (Gloo ranks, nothing on a GPU)."""
    import datetime

    import torch.distributed as dist

    g = dist.new_group(ranks=[0, 1], timeout=datetime.timedelta(seconds=2))
    t = torch.ones(1)
    if rank == 0:
        with pytest.raises(Exception):
            dist.all_reduce(t, group=g)


def test_collective_timeout_surfaces_as_error():
    try:
        run_distributed(_timeout_worker, 2, timeout=60)
    except AssertionError:
        pass   # the process group may already be torn down by the failed collective at barrier time


# ------------------------------------------------------------------ controller / schedule
def test_cadence_predicates():
    from ironcore_b200.controller import TrainingControl

    cfg = tiny_config("gpt2")
    cfg.trainer(log_interval=5, save_checkpoint_steps=10, model_path="/tmp/x", grad_norm_log_interval="log")
    cfg.operation(eval_interval=4, exit_interval=7)
    cfg.trainer.do_eval = True
    c = TrainingControl(cfg)
    assert [s for s in range(12) if c.do_log(s)] == [4, 9]
    assert [s for s in range(12) if c.do_checkpoint(s)] == [9]
    assert [s for s in range(12) if c.do_eval(s)] == [3, 7, 11]
    assert [s for s in range(12) if c.do_exit(s)] == [6]
    assert c.do_grad_norm(4) and not c.do_grad_norm(5)
    assert TrainingControl._cadence_now(10, 5) and not TrainingControl._cadence_now(0, 5)


def test_cosine_schedule_matches_documented_values():
    from ironcore_b200.optim.lr_scheduler import CosineAnnealingLR

    class Opt:
        param_groups = [{"lr": 6e-4}]

    s = CosineAnnealingLR(Opt(), max_lr=6e-4, min_lr=0.0, warmup_steps=2, annealing_steps=4, total_steps=4)
    seen = [Opt.param_groups[0]["lr"]]
    for _ in range(4):
        s.step()
        seen.append(Opt.param_groups[0]["lr"])
    # t = 1..5: warm-up 3e-4, 6e-4, then cosine over 4 steps
    assert abs(seen[0] - 3e-4) < 1e-12 and abs(seen[1] - 6e-4) < 1e-12
    assert abs(seen[2] - 6e-4 * (1 + 0.7071067811865476) / 2) < 1e-9
    assert abs(seen[3] - 3e-4) < 1e-9


# ------------------------------------------------------------------ YAML groups / CLI
def test_yaml_groups_env_and_cli(tmp_path, monkeypatch):
    from ironcore_b200.config import load_trainer_config

    (tmp_path / "model").mkdir()
    (tmp_path / "model" / "tiny.yaml").write_text(yaml.safe_dump(
        {"d_model": 64, "d_ffn": 128, "num_layers": 2, "num_attention_heads": 4, "max_seq_len": 32, "precision": "fp32"}))
    monkeypatch.setenv("MY_CKPT", str(tmp_path / "ck"))
    (tmp_path / "main.yaml").write_text(
        "model: tiny\ntrainer:\n  model_path: ${MY_CKPT}\n  micro_batch_size: 2\n  train_batch_size: 4\n"
        "optim:\n  - max_lr: 1.0e-3\n  - weight_decay: 0.1\noperation:\n  train_steps: 5\n")
    cfg = load_trainer_config(["--config-path", str(tmp_path / "main.yaml"), "--log-interval", "3", "--max_lr", "2e-3"])
    assert cfg.model.name == "tiny" and cfg.model.d_model == 64
    assert cfg.trainer.model_path == str(tmp_path / "ck")
    assert cfg.trainer.gradient_accumulation_steps == 2 and cfg.trainer.log_interval == 3
    assert cfg.optim.max_lr == 2e-3 and cfg.optim.weight_decay == 0.1
    with pytest.raises(KeyError):
        (tmp_path / "bad.yaml").write_text("nonsense:\n  a: 1\n")
        load_trainer_config(["--config-path", str(tmp_path / "bad.yaml")])


# ------------------------------------------------------------------ checkpoints under failure
def test_corrupt_and_missing_checkpoints(tmp_path):
    from ironcore_b200.checkpoint import find_latest_step, load_checkpoint, save_checkpoint
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2")
    cfg.trainer.model_path = str(tmp_path / "ck")
    validate_config(cfg)
    tr = Trainer(cfg)
    assert load_checkpoint(cfg, tr.model) == -1                    # nothing there yet
    tr.train_step(0)
    save_checkpoint(cfg, tr.model, tr.optimizer, tr.lr_scheduler, 0)
    save_checkpoint(cfg, tr.model, tr.optimizer, tr.lr_scheduler, 1)
    os.remove(tmp_path / "ck" / "latest_step.txt")
    assert find_latest_step(cfg.trainer.model_path) == 1           # falls back to scanning step_* dirs
    p = tmp_path / "ck" / "step_1" / "pytorch_model.bin"
    p.write_bytes(p.read_bytes()[:1000])                           # truncated file
    with pytest.raises(RuntimeError):
        load_checkpoint(cfg, tr.model)
    assert load_checkpoint(cfg, tr.model, step=0) == 0


# ------------------------------------------------------------------ eval task
def test_hellaswag_task_on_inline_examples():
    from ironcore_b200.config import validate_config
    from ironcore_b200.eval.tasks.hellaswag import HellaSwag
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh
    from ironcore_b200.tokenizer import Tokenizer

    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2", max_seq_len=64, max_position_embeddings=64)
    validate_config(cfg)
    model = LanguageModel(cfg).eval()
    tok = Tokenizer(512, 511, 0, 8)
    ex = [{"ctx": "a b c", "endings": ["d", "e f", "g", "hh"], "label": 1} for _ in range(3)]
    res = HellaSwag(tok, 1, None, examples=ex).process(model)
    assert res["metric"] == "accuracy" and 0.0 <= res["score"] <= 100.0


def _hellaswag_tp_worker(rank, world, out_path):
    from ironcore_b200.config import validate_config
    from ironcore_b200.eval.tasks.hellaswag import HellaSwag
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh
    from ironcore_b200.tokenizer import Tokenizer

    cfg = tiny_config("llama", max_seq_len=64, max_position_embeddings=64)
    cfg.trainer.tensor_model_parallel_size = world
    cfg.parallel(world_size=world, rank=rank)
    validate_config(cfg)
    mesh.initialize_model_parallel(world)
    torch.manual_seed(3)
    model = LanguageModel(cfg).eval()
    task = HellaSwag(Tokenizer(512, 511, 0, 8), 1, None, examples=[])
    losses = task.score_example(model, "a b c d", ["e", "f g", "hh", "i j k"])
    if rank == 0:
        torch.save(losses, out_path)


def test_hellaswag_scores_do_not_depend_on_tensor_parallel_size(tmp_path):
    """The ending losses are a softmax over the whole vocabulary: with the logits sharded over two ranks
    they must equal the single-rank values (a softmax over the local shard would not)."""
    a, b = str(tmp_path / "tp1.pt"), str(tmp_path / "tp2.pt")
    run_distributed(_hellaswag_tp_worker, 1, a)
    run_distributed(_hellaswag_tp_worker, 2, b)
    la, lb = torch.load(a), torch.load(b)
    assert torch.allclose(la, lb, atol=1e-4), (la, lb)


def test_gpt2_loss_curve_matches_reference_cpu():
    """Same weights, same batches, same optimizer settings: the loss curve of the unmodified reference
    trainer and ours agree step by step (fp32, CPU). Runs in a child process because the reference
    owns its own process group and global state."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.isdir(os.path.join(root, "baseline", "_ref", "ironcore")):
        pytest.skip("reference is not installed under baseline/_ref")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-m", "baseline.parity_gpt2", "--layers", "2", "--d-model", "64", "--heads",
                          "4", "--vocab", "512", "--seq", "32", "--micro-batch", "2", "--steps", "8"],
                         cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["missing_in_ours"] == [] and res["not_in_ours"] == []
    assert res["max_abs_diff"] < 1e-4, res


def test_examples_run_on_cpu(tmp_path):
    """The flag-driven training example and the text-generation example run end to end on CPU."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    flags = ("--model_name tiny --name llama --d_model 64 --d_ffn 128 --num_layers 2 --num_attention_heads 4 "
             "--max_seq_len 32 --max_position_embeddings 32 --precision fp32 --ln_type rmsnorm --activation_type swiglu "
             "--task_type synthetic --vocab_size 512 --train_steps 2 --no_save true --micro_batch_size 2 "
             "--train_batch_size 4 --log_interval 1 --dist_backend gloo").split()
    out = subprocess.run([sys.executable, os.path.join(root, "examples", "train.py"), *flags], cwd=tmp_path, env=env,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "step      2" in out.stdout + out.stderr
    cfg = tmp_path / "gen.yaml"
    cfg.write_text("trainer: {micro_batch_size: 1, train_batch_size: 1, model_path: ''}\noperation: {no_save: true}\n"
                   "model: {name: llama, d_model: 64, d_ffn: 128, num_layers: 2, num_attention_heads: 4, max_seq_len: 64,\n"
                   "  max_position_embeddings: 64, precision: fp32, ln_type: rmsnorm, activation_type: swiglu, vocab_size: 300,\n"
                   "  tokenizer_type: byte, vocab_name_or_path: none, positional_embedding: {type: rope}}\n"
                   "data: {task_type: synthetic, vocab_size: 300}\nparallel: {dist_backend: gloo}\n")
    out = subprocess.run([sys.executable, os.path.join(root, "examples", "generate_text.py"), "--config", str(cfg),
                          "--prompt", "hello", "--max-new-tokens", "6"], cwd=tmp_path, env=env, capture_output=True,
                         text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "--- sample 0 ---" in out.stdout


def test_constructed_baselines_run_tiny_on_cpu():
    """The plain-PyTorch baselines of the MoE, FSDP+Muon and GRPO workloads execute end to end (tiny shapes)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    for workload in ("moe", "fsdp_muon", "grpo"):
        out = subprocess.run([sys.executable, "-m", "baseline.constructed", "--workload", workload, "--tiny",
                              "--steps", "1", "--warmup", "1"], cwd=root, env=env, capture_output=True, text=True,
                             timeout=300)
        assert out.returncode == 0, out.stderr[-1500:]
        line = json.loads(out.stdout.strip().splitlines()[-1])
        assert line["workload"] == workload and line["value"] > 0


# ------------------------------------------------------------------ tracing
def test_torch_profiler_window_stops_training_and_writes_a_trace(tmp_path):
    """``utils.profile_torch``: the profiler runs over [profile_step_start, profile_step_end), training stops when
    the window ends, a trace lands under ``utils.tensorboard_dir`` and no final checkpoint is written."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2")
    cfg.trainer.model_path = str(tmp_path / "ck")
    cfg.operation.train_steps = 10
    cfg.utils(profile_torch=True, profile_step_start=1, profile_step_end=3, tensorboard_dir=str(tmp_path / "tb"),
              profile_ranks=[0])
    validate_config(cfg)
    tr = Trainer(cfg)
    last = tr.train()
    assert last == 2                                   # steps 0, 1, 2 ran; the window ended at step 3
    traces = [p for p in (tmp_path / "tb").rglob("*") if p.is_file() and "trace" in p.name]
    assert traces, list((tmp_path / "tb").rglob("*"))
    assert not (tmp_path / "ck").exists() or not any((tmp_path / "ck").glob("step_*"))


def test_module_profile_hooks_put_ranges_into_a_trace():
    """``BaseModule.register_profile_hooks``: every submodule's forward and backward appear as named ranges."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.models.language_model import LanguageModel
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = tiny_config("gpt2")
    validate_config(cfg)
    model = LanguageModel(cfg)
    model.register_profile_hooks(profile_torch=True, profile_nsys=False)
    ids = torch.randint(0, 512, (2, 16))
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        model(ids, ids).backward()
    names = {e.key for e in prof.key_averages()}
    assert any(n.startswith("Forward TransformerLayer") for n in names), sorted(names)[:20]
    assert any(n.startswith("Forward MLP") for n in names)
    model.remove_profile_hooks()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        model(ids, ids)
    assert not any(e.key.startswith("Forward TransformerLayer") for e in prof.key_averages())


def test_special_tokens_file_reaches_the_tokenizer(tmp_path):
    """``trainer.special_tokens_config_path`` (looked up under the vocabulary / model path) overrides the special
    ids the model and the data pipeline use."""
    import json

    from ironcore_b200.config import validate_config
    from ironcore_b200.global_vars import set_global_states

    (tmp_path / "special_tokens.json").write_text(json.dumps({"eos_token": "</s>", "eos_token_id": 2, "pad_token_id": 1}))
    cfg = tiny_config("gpt2")
    cfg.trainer(special_tokens_config_path="special_tokens.json", model_path=str(tmp_path))
    validate_config(cfg)
    assert cfg.data.special_tokens["eos_token_id"] == 2
    tok = set_global_states(cfg).tokenizer
    assert (tok.eos_token_id, tok.eod_token_id, tok.pad_token_id, tok.eos_token) == (2, 2, 1, "</s>")
    assert (cfg.model.eod_token_id, cfg.model.pad_token_id) == (2, 1)
    cfg2 = tiny_config("gpt2")
    cfg2.trainer(special_tokens_config_path="missing.json", model_path=str(tmp_path))
    with pytest.raises(FileNotFoundError):
        validate_config(cfg2)
