"""End-to-end trainer on CPU (fp32): the loss falls, checkpoints resume, config derivation works."""

import pytest
import torch

from helpers import tiny_config


def _run(cfg):
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    validate_config(cfg)
    tr = Trainer(cfg)
    losses = []
    for step in range(cfg.operation.train_steps):
        loss, gn, _ = tr.train_step(step)
        losses.append(float(loss))
    return tr, losses


def test_gpt2_tiny_trains():
    cfg = tiny_config("gpt2")
    cfg.operation.train_steps = 8
    cfg.optim.max_lr = 3e-3
    # repeat the same batch so the loss must fall
    from ironcore_b200.data.synthetic import SyntheticTokenStream

    tr, _ = None, None
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    validate_config(cfg)
    batch = next(SyntheticTokenStream(512, 32, 2, seed=1, pin=False))

    def it():
        while True:
            yield batch

    tr = Trainer(cfg, data_iterator={"train": it(), "eval": None, "test": None})
    losses = [float(tr.train_step(s)[0]) for s in range(8)]
    assert losses[-1] < losses[0] - 0.5, losses


def test_llama_tiny_trains_and_resumes(tmp_path):
    cfg = tiny_config("llama")
    cfg.trainer.model_path = str(tmp_path / "ckpt")
    cfg.trainer.save_checkpoint_steps = 2
    cfg.operation.train_steps = 4
    from ironcore_b200.config import validate_config
    from ironcore_b200.trainer import Trainer

    validate_config(cfg)
    tr = Trainer(cfg)
    assert tr.train() == 3
    w_ref = {k: v.clone() for k, v in tr.model.state_dict().items()}
    assert (tmp_path / "ckpt" / "latest_step.txt").read_text() == "3"
    # resume into a fresh trainer: weights and optimizer state come back
    cfg2 = tiny_config("llama")
    cfg2.trainer.model_path = cfg.trainer.model_path
    cfg2.operation.train_steps = 4
    validate_config(cfg2)
    tr2 = Trainer(cfg2)
    from ironcore_b200.checkpoint import load_checkpoint

    assert load_checkpoint(cfg2, tr2.model, tr2.optimizer, tr2.lr_scheduler) == 3
    for k, v in tr2.model.state_dict().items():
        assert torch.equal(v, w_ref[k]), k
    assert tr2.optimizer.step_count == tr.optimizer.step_count
    m1 = tr.optimizer.moments[0]["exp_avg"]
    m2 = tr2.optimizer.moments[0]["exp_avg"]
    assert torch.allclose(m1, m2)


def test_batch_derivation_and_validation():
    import pytest

    from ironcore_b200.config import validate_config

    cfg = tiny_config("gpt2")
    cfg.trainer(micro_batch_size=2, train_batch_size=8, gradient_accumulation_steps=None)
    validate_config(cfg)
    assert cfg.trainer.gradient_accumulation_steps == 4
    cfg.trainer(micro_batch_size=3)
    with pytest.raises(ValueError):
        validate_config(cfg)


def test_param_norm_over_flat_buffers_matches_per_tensor_loop():
    from helpers import tiny_config
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    mesh.destroy_model_parallel()
    cfg = tiny_config("llama")
    validate_config(cfg)
    tr = Trainer(cfg)
    want = torch.sqrt(sum(p.detach().float().pow(2).sum() for p in tr.model.parameters()))
    got = tr._param_norm()
    assert torch.allclose(got, want, rtol=1e-5), (float(got), float(want))


def test_lm_head_chunk_gives_the_same_loss_and_gradients():
    """``model.lm_head_chunk``: the loss and every gradient of a small model equal the materialised-logits path,
    tied and untied heads."""
    from helpers import tiny_config
    from ironcore_b200.models.language_model import LanguageModel
    from ironcore_b200.parallel import mesh

    for untie in (False, True):
        grads = []
        for chunk in (0, 128):
            mesh.destroy_model_parallel()
            cfg = tiny_config("llama", d_model=64, d_ffn=128, num_layers=2, num_attention_heads=4, head_dim=16,
                              max_seq_len=32, max_position_embeddings=32, vocab_size=300)
            cfg.data.vocab_size = 300
            cfg.model(untie_embed=untie, lm_head_chunk=chunk)
            torch.manual_seed(11)
            model = LanguageModel(cfg)
            ids = torch.randint(0, 300, (2, 32))
            labels = torch.roll(ids, -1, dims=1)
            labels[0, -1] = -100
            loss = model(ids, labels)
            loss.backward()
            grads.append((loss.detach(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}))
        (la, ga), (lb, gb) = grads
        assert torch.allclose(la, lb, atol=1e-5), (untie, la, lb)
        assert ga.keys() == gb.keys()
        for n in ga:
            assert torch.allclose(ga[n], gb[n], atol=2e-5, rtol=1e-4), (untie, n)


def test_evaluation_reports_the_loss_of_the_counted_positions():
    """``Trainer.evaluate`` / ``test``: one forward pass per batch; loss, perplexity and arg-max accuracy over the
    positions the training loss counts (SFT masks and sample boundaries included)."""
    import math

    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    mesh.destroy_model_parallel()
    cfg = tiny_config("llama")
    cfg.trainer(do_eval=True, do_test=True, eval_batch_size=2, test_batch_size=2)
    cfg.operation(eval_samples=4, test_samples=2)
    validate_config(cfg)
    tr = Trainer(cfg)
    m = tr.evaluate(0)
    assert set(m) == {"eval_loss", "eval_ppl", "eval_accuracy"}
    assert m["eval_ppl"] == pytest.approx(math.exp(m["eval_loss"]), rel=1e-6) and 0.0 <= m["eval_accuracy"] <= 1.0
    assert abs(m["eval_loss"] - math.log(512)) < 0.5                    # an untrained model on uniform tokens
    assert set(tr.test(0)) == {"test_loss", "test_ppl", "test_accuracy"}

    # a packed SFT batch: only unmasked answer tokens count, attention stays inside each sample
    ids = torch.randint(1, 500, (1, 32))
    labels = torch.roll(ids, -1, dims=1)
    labels[:, :10] = -100
    labels[:, 20:] = -100
    batch = {"input_ids": ids, "labels": labels, "position_ids": torch.cat([torch.arange(16), torch.arange(16)])[None],
             "cu_seqlens": torch.tensor([0, 16, 32], dtype=torch.int32), "loss_mask": labels != -100}
    got = tr._eval_loop(iter([batch]), 1, "eval", 0)
    tr.model.eval()
    with torch.no_grad():
        want = float(tr.model(ids, labels, position_ids=batch["position_ids"], cu_seqlens=batch["cu_seqlens"],
                              loss_mask=batch["loss_mask"]))
        logits = tr.model(ids, position_ids=batch["position_ids"], cu_seqlens=batch["cu_seqlens"])
    keep = labels != -100
    acc = float(((logits.argmax(-1) == labels) & keep).sum()) / float(keep.sum())
    assert got["eval_loss"] == pytest.approx(want, rel=1e-5) and got["eval_accuracy"] == pytest.approx(acc)


def test_interrupted_run_continues_as_if_uninterrupted(tmp_path):
    """Two steps, a checkpoint, a new process-worth of objects, two more steps: the same weights as four steps in
    one go. Weights, optimizer state, schedule and the position in the data stream all come back."""
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    def run(steps, path, accum=2):
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama")
        cfg.trainer(micro_batch_size=2, train_batch_size=2 * accum, gradient_accumulation_steps=None, model_path=path,
                    save_checkpoint_steps=100)
        cfg.optim(lr_scheduler="cosine", warmup_steps=1, annealing_steps=10, max_lr=1e-3)
        cfg.operation(train_steps=steps)
        validate_config(cfg)
        tr = Trainer(cfg)
        last = tr.train()
        return last, {k: v.clone() for k, v in tr.model.canonical_state_dict().items()}

    last, whole = run(4, str(tmp_path / "a"))
    assert last == 3
    last, _ = run(2, str(tmp_path / "b"))            # ends with the final checkpoint of step 1
    assert last == 1
    last, resumed = run(4, str(tmp_path / "b"))      # picks it up and goes on to step 3
    assert last == 3
    for k, v in whole.items():
        assert torch.equal(v, resumed[k]), k
