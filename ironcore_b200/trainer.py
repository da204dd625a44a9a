"""Training orchestration: process / mesh bootstrap, data, model, optimizer engine, the
step loop with gradient accumulation, logging (loss, lr, norms, tokens/s, MFU), evaluation,
checkpoint cadence, profiling windows and failure detection.

``Trainer(config, forward_step_func, loss_fn)`` with ``.train()``, ``.train_step(step)``,
``.evaluate()``, ``.evaluate_subtask()``, ``.test()``; usable as a context manager.
(Behavioural reference: ironcore/trainer.py:55-549. Differences by design: evaluation and
exit checks run on their own cadence rather than only on checkpoint steps; the logged loss
is averaged over the data-parallel group size.)
"""

from __future__ import annotations

import json
import math
import os
import random
from typing import Callable, Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import global_vars as G
from .controller import TrainingControl
from .data import get_data_iterator
from .models.language_model import LanguageModel, get_model_dtype
from .optim import get_lr_scheduler, get_optimizer
from .parallel import mesh
from .training_utils import compute_token_accuracy, forward_step as default_forward_step, get_loss_func
from .utils.timers import DeviceTimer, get_memory_usage


def model_flops_per_token(config) -> float:
    """Training FLOPs per token (forward + backward = 3x forward) of the configured model."""
    m = config.model
    d, L, s = m.d_model, m.num_layers, m.max_seq_len
    hd = m.head_dim or (d // m.num_attention_heads)
    hq, hkv = m.num_attention_heads, (m.num_attention_groups or m.num_attention_heads)
    from .layers.activations import is_glu

    ffn_mult = 3 if is_glu(m.activation_type) else 2
    per_layer = 2 * d * (hq + 2 * hkv) * hd + 2 * hq * hd * d
    if m.moe.num_experts > 0:
        e_ffn = m.moe.expert_d_ffn or m.d_ffn
        s_ffn = (m.moe.shared_expert_d_ffn or e_ffn) * m.moe.num_shared_experts
        per_layer += 2 * d * (e_ffn * m.moe.top_k + s_ffn) * ffn_mult + 2 * d * m.moe.num_experts
    else:
        per_layer += 2 * d * m.d_ffn * ffn_mult
    attn = 2 * 2 * s * hq * hd / 2  # causal: half of the s x s score / value products
    vocab = m.padded_vocab_size or m.vocab_size or config.data.vocab_size
    return 3.0 * (L * (per_layer + attn) + 2 * d * vocab)


class Trainer:
    def __init__(self, config, forward_step_func: Optional[Callable] = None, loss_fn: Optional[Callable] = None,
                 data_iterator: Optional[Dict] = None, tokenizer=None):
        self.config = config
        if config.parallel.rank < 0:
            config.parallel.rank = int(os.environ.get("RANK", "0"))
        G.set_global_states(config, tokenizer=tokenizer)
        self.timer = G.get_timer()
        self.logger = G.get_logger()
        self.forward_step_func = forward_step_func or default_forward_step
        self.loss_fn = loss_fn or get_loss_func(getattr(config.data, "task_type", "pretrain"))
        self.control = TrainingControl(config)

        mesh.initialize_process(config)
        mesh.initialize_model_parallel(
            config.trainer.tensor_model_parallel_size,
            expert_model_parallel_size=config.parallel.expert_model_parallel_size,
            sequence_parallel=config.parallel.sequence_parallel,
            timeout_in_minutes=float(config.parallel.timeout_minute or 10.0),
        )
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
        self.data_iterator = data_iterator if data_iterator is not None else get_data_iterator(config)
        self.evaluators = []
        if config.trainer.do_eval_subtask:
            from .eval import get_evaluators

            self.evaluators = get_evaluators(config.data.eval_datasets, config.trainer.eval_batch_size,
                                             config.operation.eval_samples)
        self.model, self.optimizer = self._build_model_and_optimizer()
        self.lr_scheduler = get_lr_scheduler(config, self.optimizer)
        self.profiler = None
        self.heartbeat = None
        if config.utils.heartbeat_interval_s > 0 and dist.is_initialized():
            from .parallel.fault import Heartbeat

            self.heartbeat = Heartbeat(interval_s=config.utils.heartbeat_interval_s,
                                       timeout_s=config.utils.heartbeat_timeout_s)
        self.tokens_per_step = config.trainer.train_batch_size * config.model.max_seq_len
        self._flops_per_token = model_flops_per_token(config)
        self._step_timer = DeviceTimer() if self.device.type == "cuda" else None
        self._memory_reported = False
        self.last_step = -1
        # CUDA-graph replay of the micro-batch (forward + backward): removes the host launch cost of
        # the ~2000 kernels of a micro-batch, which dominates once tensor parallelism shrinks them.
        self._graph_enabled = bool(config.trainer.cuda_graph) and self.device.type == "cuda" \
            and self.forward_step_func is default_forward_step and not config.parallel.use_fsdp
        if self._graph_enabled and (config.model.reset_attention_mask or config.model.reset_position_ids) \
                and config.model.eod_token_id is not None:
            self.logger.warning("trainer.cuda_graph is off: document-boundary resets need a host-side scan per batch")
            self._graph_enabled = False
        self._graph = None
        self._graph_stream = None
        self._graph_eager_done = 0
        self._graph_launches = 0

    # ------------------------------------------------------------------ lifecycle
    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.finalize()

    def finalize(self):
        G.global_states_cleanup()
        if self._graph is not None:
            # a captured graph keeps NCCL work objects alive: drop it before the process group goes away
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._graph = None
            self._static_loss = None
            import gc

            gc.collect()
        if self.heartbeat is not None:
            self.heartbeat.stop()
        if dist.is_initialized():
            mesh.finalize_process()

    def _seed_everything(self):
        seed = int(self.config.init.seed)
        if self.config.init.data_parallel_random_init:
            seed += 100 * mesh.get_data_parallel_rank()
        random.seed(seed)
        np.random.seed(seed % (2 ** 32))
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    def _build_model_and_optimizer(self):
        cfg = self.config
        self._seed_everything()
        from .parallel.symmetric import configure as configure_comm_policy

        configure_comm_policy(cfg.parallel)
        dtype = get_model_dtype(cfg)
        if self.device.type == "cpu" and dtype != torch.float32:
            self.logger.warning("16-bit precision on CPU runs the PyTorch reference path")
        model = LanguageModel(cfg, self.loss_fn, device=self.device)
        if cfg.parallel.use_fsdp:
            from .parallel.fsdp import FullyShardedModel

            model = FullyShardedModel(model, cfg)
            optimizer = model.build_optimizer()
        else:
            optimizer = get_optimizer(cfg, model, self.device.type)
        if cfg.parallel.fused_comm and self.device.type == "cuda" and mesh.get_tensor_model_parallel_world_size() > 1 \
                and mesh.sequence_parallel_enabled():
            from .parallel.fused_comm import attach_fused_tp

            self.fused_tp = attach_fused_tp(model, cfg)
        if cfg.utils.profile_torch or cfg.utils.profile_nsys:
            base = model.module if hasattr(model, "module") else model
            if hasattr(base, "register_profile_hooks"):
                base.register_profile_hooks(use_nvtx=cfg.utils.profile_nsys, use_record_function=cfg.utils.profile_torch)
        n_params = sum(p.numel() for p in model.parameters())
        self.logger.info("model %s: %.1fM parameters on this rank (%s)", cfg.model.name, n_params / 1e6, dtype)
        return model, optimizer

    def load_or_init_weights(self) -> int:
        """Resume from the latest checkpoint under ``trainer.model_path`` (weights, optimizer, schedule) and return
        the step to continue at; without one start at step 0, from the HuggingFace checkpoint named by
        ``trainer.init_from_hf`` when that is set, else from the random initialisation."""
        from .checkpoint import load_checkpoint

        cfg = self.config
        last = load_checkpoint(cfg, self.model, self.optimizer, self.lr_scheduler)
        if last is not None and last >= 0:
            if cfg.operation.resume_data_position:
                # the stream is seeded and deterministic: the completed steps consumed this many micro-batches
                self._skip_training_batches((last + 1) * int(cfg.trainer.gradient_accumulation_steps))
            return last + 1
        if cfg.trainer.init_from_hf:
            from .checkpoint.hf_interop import load_from_huggingface

            load_from_huggingface(self.model, cfg, cfg.trainer.init_from_hf)
            self.logger.info("initialised the weights from the HuggingFace checkpoint %s", cfg.trainer.init_from_hf)
        return 0

    def _skip_training_batches(self, n: int) -> None:
        it = self.data_iterator.get("train") if isinstance(self.data_iterator, dict) else None
        if it is None or n <= 0:
            return
        if hasattr(it, "skip_batches"):      # file-backed streams move their starting point without reading tokens
            it.skip_batches(n)
            return
        for _ in range(n):
            try:
                next(it)
            except StopIteration:
                break

    # ------------------------------------------------------------------ training
    def train(self):
        cfg = self.config
        from .checkpoint import save_checkpoint

        step = self.load_or_init_weights()
        self._start_profiler()
        loss_acc, n_acc = 0.0, 0
        pending = []
        while step < cfg.operation.train_steps:
            if self._profile_tick(step):
                break
            if self.heartbeat is not None:
                self.heartbeat.beat(step)
                self.heartbeat.raise_if_peer_dead()
            try:
                loss, grad_norm, param_norm = self.train_step(step)
            except BaseException as e:
                if self.heartbeat is not None:     # the peers stop before their next step instead of waiting for us
                    self.heartbeat.leave(f"{type(e).__name__}: {e}")
                raise
            pending.append(loss)
            if self.control.do_log(step):
                self.log_training(step, pending, grad_norm, param_norm)
                pending = []
            if self.control.do_checkpoint(step):
                save_checkpoint(cfg, self.model, self.optimizer, self.lr_scheduler, step)
            if self.control.do_eval(step):
                self.evaluate(step)
            if self.control.do_eval_subtask(step):
                self.evaluate_subtask(step)
            self.last_step = step
            if self.control.do_exit(step):
                self.logger.info("exit_interval reached at step %d", step)
                break
            step += 1
        self._stop_profiler()
        if self.control.do_final_checkpoint() and self.last_step >= 0 \
                and not self.control.do_checkpoint(self.last_step):
            save_checkpoint(cfg, self.model, self.optimizer, self.lr_scheduler, self.last_step)
        if cfg.trainer.do_test:
            self.test()
        return self.last_step

    def train_step(self, step: int):
        """One optimizer step over ``gradient_accumulation_steps`` micro-batches. Returns
        (mean loss tensor, grad norm tensor or None, param norm tensor or None); nothing here
        forces a device synchronisation."""
        cfg = self.config
        accum = cfg.trainer.gradient_accumulation_steps
        self.model.train()
        self.timer.start("iter")
        if self._step_timer is not None:
            self._step_timer.start()
        total = None
        if self._graph_enabled:
            # Everything of the micro-batch loop (eager warm-up, capture, replays) runs on one side
            # stream: gradient-accumulation nodes remember the stream they were created on, and a node
            # created on the legacy default stream cannot take part in a capture.
            if self._graph_stream is None:
                self._graph_stream = torch.cuda.Stream()
            main = torch.cuda.current_stream()
            self._graph_stream.wait_stream(main)
            with torch.cuda.stream(self._graph_stream):
                for _ in range(accum):
                    loss = self._graphed_micro_batch(accum)
                    total = loss.detach().clone() if total is None else total + loss.detach()
            main.wait_stream(self._graph_stream)
        else:
            overlap = getattr(self.optimizer, "start_grad_reduce_overlap", None)
            for i in range(accum):
                if i == accum - 1 and overlap is not None:
                    overlap()   # gradient buckets are reduced behind this micro-batch's backward pass
                loss = self.forward_step_func(self.model, self.data_iterator["train"])
                (loss / accum).backward()
                total = loss.detach() if total is None else total + loss.detach()
        grad_norm = self.optimizer.step()
        self.optimizer.zero_grad()
        self.lr_scheduler.step()
        param_norm = None
        if self.control.do_param_norm(step):
            param_norm = self._param_norm()
        if self._step_timer is not None:
            self._step_timer.stop()
        self.timer.stop("iter")
        return total / accum, grad_norm, param_norm

    def _graphed_micro_batch(self, accum: int):
        """Two eager micro-batches (allocator / lazy-init warm-up), then capture once and replay."""
        from .ops import native

        batch = next(self.data_iterator["train"])
        extra = [k for k in batch if k not in ("input_ids", "labels") and batch[k] is not None]
        if extra:
            raise RuntimeError(f"trainer.cuda_graph supports (input_ids, labels) batches only, got extra {extra}")
        if self._graph is None and self._graph_eager_done < 2:
            self._graph_eager_done += 1
            loss = self.model(batch["input_ids"], batch["labels"])
            (loss / accum).backward()
            return loss
        if self._graph is None:
            self._static_ids = batch["input_ids"].to(self.device).clone()
            self._static_labels = batch["labels"].to(self.device).clone()
            ws = None
            for m in self.model.modules():
                cand = getattr(m, "fused", None)
                if cand is not None and hasattr(cand, "g_epoch") and hasattr(cand, "r_epoch"):
                    ws = cand
                    break
            before = (ws.g_epoch, ws.r_epoch) if ws is not None else (0, 0)
            count0 = native.launches()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self._graph_stream):
                loss = self.model(self._static_ids, self._static_labels)
                (loss / accum).backward()
                self._static_loss = loss.detach()
            if ws is not None and (((ws.g_epoch - before[0]) | (ws.r_epoch - before[1])) & 1):
                raise RuntimeError("a captured micro-batch must issue an even number of fused gather / scatter "
                                   "calls (buffer parity is fixed at capture time)")
            self._graph_launches = native.launches() - count0
            self._graph = graph
        else:
            self._static_ids.copy_(batch["input_ids"], non_blocking=True)
            self._static_labels.copy_(batch["labels"], non_blocking=True)
            native.add_launches(self._graph_launches)
        self._graph.replay()
        return self._static_loss

    def _param_norm(self):
        fused = getattr(self.optimizer, "param_norm", None)
        if fused is not None:
            return fused()
        sq = None
        for p in self.model.parameters():
            v = p.detach().float().pow(2).sum()
            sq = v if sq is None else sq + v
        return sq.sqrt() if sq is not None else None

    def average_loss(self, losses) -> float:
        """Mean of the pending step losses, averaged over the data-parallel group."""
        t = torch.stack([l.float() for l in losses]).mean()
        dp = mesh.get_data_parallel_world_size()
        if dp > 1:
            dist.all_reduce(t, group=mesh.get_data_parallel_group())
            t = t / dp
        return float(t.item())

    def log_training(self, step: int, losses, grad_norm, param_norm):
        cfg = self.config
        loss = self.average_loss(losses)
        if self._step_timer is not None:
            ms = self._step_timer.elapsed_ms()
            iter_s = (sum(ms) / len(ms) / 1e3) if ms else self.timer.elapsed("iter")
        else:
            iter_s = self.timer.elapsed("iter", reset=True)
        lr = self.optimizer.param_groups[0]["lr"]
        tok_s = self.tokens_per_step / iter_s if iter_s > 0 else 0.0
        metrics = {"lm_loss": loss, "lr": lr, "tokens_per_s": tok_s}
        peak = _measured_bf16_peak()
        if peak and self.device.type == "cuda":
            world = mesh.get_world_size()
            metrics["mfu"] = tok_s * self._flops_per_token / (peak * 1e12 * world)
        msg = f"step {step + 1:6d} | loss {loss:.4f}"
        if grad_norm is not None and self.control.do_grad_norm(step):
            gn = float(grad_norm.item()) if torch.is_tensor(grad_norm) else float(grad_norm)
            metrics["grad_norm"] = gn
            msg += f" | grad norm {gn:.3f}"
        if param_norm is not None:
            pn = float(param_norm.item())
            metrics["param_norm"] = pn
            msg += f" | param norm {pn:.3f}"
        msg += f" | iter {iter_s * 1e3:.1f} ms | {tok_s:,.0f} tok/s | lr {lr:.3e}"
        if "mfu" in metrics:
            msg += f" | MFU {100 * metrics['mfu']:.1f}%"
        self.logger.info(msg)
        G.log_metrics(metrics, step + 1)
        if cfg.utils.report_memory_usage and not self._memory_reported:
            mem = get_memory_usage()
            self.logger.info("memory (MiB): allocated %.0f | reserved %.0f | peak %.0f", mem["allocated"],
                             mem["reserved"], mem["max_allocated"])
            self._memory_reported = True
        if self.device.type == "cuda":
            from .ops import native

            native.check_status()
        return metrics

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def _eval_loop(self, iterator, max_batches: int, tag: str, step: int):
        if iterator is None:
            return None
        self.model.eval()
        losses, accs = [], []
        for i, batch in enumerate(iterator):
            if i >= max_batches:
                break
            ids, labels = batch["input_ids"], batch["labels"]
            extra = {k: batch[k] for k in ("position_ids", "cu_seqlens") if batch.get(k) is not None}
            if hasattr(self.model, "compute_loss_from_logits"):
                # one forward pass: loss and accuracy from the same logits, on the positions the training loss counts
                logits = self.model(ids, **extra)
                ids, labels = ids.to(logits.device), labels.to(logits.device)
                mask = self.model._loss_mask(ids, labels, batch.get("loss_mask"))   # pylint: disable=protected-access
                losses.append(self.model.compute_loss_from_logits(logits, labels, mask).float())
            else:   # a wrapper that only exposes forward (FSDP): loss and logits from two passes
                losses.append(self.model(ids, labels, **extra).float())
                logits = self.model(ids, **extra)
                mask = None
            accs.append(compute_token_accuracy(logits, labels.to(logits.device), mask))
        self.model.train()
        if not losses:
            return None
        loss = self.average_loss(losses)
        metrics = {f"{tag}_loss": loss, f"{tag}_ppl": math.exp(min(loss, 30.0)),
                   f"{tag}_accuracy": sum(accs) / len(accs)}
        self.logger.log_metrics(metrics, title=f"{tag} @ step {step + 1}")
        G.log_metrics(metrics, step + 1)
        return metrics

    def evaluate(self, step: int = 0):
        bs = self.config.trainer.eval_batch_size or self.config.trainer.micro_batch_size
        n = max(1, self.config.operation.eval_samples // max(bs, 1))
        return self._eval_loop(self.data_iterator.get("eval"), n, "eval", step)

    def test(self, step: Optional[int] = None):
        bs = self.config.trainer.test_batch_size or self.config.trainer.micro_batch_size
        n = max(1, self.config.operation.test_samples // max(bs, 1))
        return self._eval_loop(self.data_iterator.get("test"), n, "test", self.last_step if step is None else step)

    @torch.no_grad()
    def evaluate_subtask(self, step: int = 0):
        out = {}
        self.model.eval()
        for task in self.evaluators:
            res = task.process(self.model)
            name = f"{task.name}/{res['metric']}"
            out[name] = res["score"]
            G.log_metric(name, res["score"], step + 1)
        self.model.train()
        if out:
            self.logger.log_metrics(out, title=f"subtasks @ step {step + 1}")
        return out

    # ------------------------------------------------------------------ profiling windows
    def _start_profiler(self):
        u = self.config.utils
        if u.profile_torch and (u.profile_ranks is None or mesh.get_rank() in u.profile_ranks):
            start, end = int(u.profile_step_start or 1), int(u.profile_step_end or 2)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            handler = None
            if u.tensorboard_dir:
                handler = torch.profiler.tensorboard_trace_handler(u.tensorboard_dir)
            self.profiler = torch.profiler.profile(
                activities=acts, schedule=torch.profiler.schedule(wait=1, warmup=max(start - 1, 0),
                                                                  active=max(end - start, 1)),
                on_trace_ready=handler, record_shapes=True, with_stack=True, profile_memory=True, with_flops=True)
            self.profiler.start()

    def _profile_tick(self, step: int) -> bool:
        """Advance profiling windows; returns True when training should stop (window ended)."""
        u = self.config.utils
        if self.profiler is not None:
            self.profiler.step()
            if step >= int(u.profile_step_end or 0):
                return True
        if u.profile_nsys and torch.cuda.is_available():
            if step == int(u.profile_step_start or 0):
                torch.cuda.profiler.start()
            if step >= int(u.profile_step_end or 0):
                torch.cuda.profiler.stop()
                return True
        return False

    def _stop_profiler(self):
        if self.profiler is not None:
            self.profiler.stop()
            self.profiler = None


_PEAK = None


def _measured_bf16_peak() -> Optional[float]:
    """Sustained bf16 GEMM TFLOP/s measured on this machine pool, if a measurement file is
    present at the repository root (``MEASURED_PEAKS.json``)."""
    global _PEAK
    if _PEAK is None:
        _PEAK = 0.0
        here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        path = os.path.join(here, "MEASURED_PEAKS.json")
        try:
            with open(path) as f:
                doc = json.load(f)
            _PEAK = float(doc.get("bf16_tflops_sustained") or doc.get("bf16_tflops") or 0.0)
        except Exception:
            _PEAK = 0.0
    return _PEAK or None
