"""Configuration schema: one dataclass per YAML group.

Field names and defaults follow the reference project's public configuration
surface (reference: ironcore/config/config_model.py, config_trainer.py,
config_optim.py, config_parallel.py, config_utils.py, config_data.py) so existing
YAML files load unchanged. Groups and fields the reference lacks (sequence /
expert parallelism, ZeRO, MoE, Muon, RL rollouts, CPU offload) are added here.
"""

from __future__ import annotations

import typing
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Dict, List, Literal, Optional, Union

import yaml


def _type_ok(value: Any, tp: Any) -> bool:
    """Structural type check for the subset of typing constructs used by the schema."""
    if tp is Any:
        return True
    origin = typing.get_origin(tp)
    if origin is Union:
        return any(_type_ok(value, a) for a in typing.get_args(tp))
    if origin is Literal:
        return value in typing.get_args(tp)
    if origin in (list, List):
        if not isinstance(value, (list, tuple)):
            return False
        args = typing.get_args(tp)
        return all(_type_ok(v, args[0]) for v in value) if args else True
    if origin in (dict, Dict):
        return isinstance(value, dict)
    if tp is type(None):
        return value is None
    if tp is float:
        return isinstance(value, (int, float)) and not isinstance(value, bool)
    if tp is int:
        return isinstance(value, int) and not isinstance(value, bool)
    if is_dataclass(tp):
        return isinstance(value, (tp, dict))
    if isinstance(tp, type):
        return isinstance(value, tp)
    return True


def _coerce(value: Any, tp: Any) -> Any:
    """Light coercions YAML needs: '6.0e-4' strings for floats, ints for floats."""
    origin = typing.get_origin(tp)
    if origin is Union:
        args = typing.get_args(tp)
        if value is None and type(None) in args:
            return None
        for a in args:
            if a is type(None):
                continue
            try:
                c = _coerce(value, a)
            except (TypeError, ValueError):
                continue
            if _type_ok(c, a):
                return c
        return value
    if tp is float and isinstance(value, str):
        return float(value)
    if tp is float and isinstance(value, int) and not isinstance(value, bool):
        return float(value)
    if tp is int and isinstance(value, str):
        return int(value.replace("_", ""))
    if tp is bool and isinstance(value, str):
        if value.lower() in ("true", "1", "yes"):
            return True
        if value.lower() in ("false", "0", "no"):
            return False
    return value


class BaseConfig:
    """Mixin for all config groups: in-place typed update, dict / YAML round trip."""

    def __call__(self, **kwargs):
        return self.update(**kwargs)

    def update(self, **kwargs):
        hints = typing.get_type_hints(type(self))
        known = {f.name for f in fields(self)}
        for key, value in kwargs.items():
            if key not in known:
                raise KeyError(f"{type(self).__name__} has no option '{key}'")
            tp = hints[key]
            current = getattr(self, key)
            if is_dataclass(current) and isinstance(value, dict):
                current.update(**value)
                continue
            value = _coerce(value, tp)
            if not _type_ok(value, tp):
                raise TypeError(f"{type(self).__name__}.{key}: expected {tp}, got {type(value).__name__} ({value!r})")
            setattr(self, key, value)
        return self

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            out[f.name] = v.to_dict() if isinstance(v, BaseConfig) else v
        for k, v in self.__dict__.items():  # free-form extras (data group)
            if k not in out and not k.startswith("_"):
                out[k] = v
        return out

    def to_yaml(self, path: Optional[str] = None) -> str:
        text = yaml.safe_dump(self.to_dict(), sort_keys=False)
        if path is not None:
            with open(path, "w") as f:
                f.write(text)
        return text

    @classmethod
    def from_dict(cls, data: Dict[str, Any]):
        obj = cls()
        obj.update(**{k: v for k, v in data.items()})
        return obj

    @classmethod
    def from_yaml(cls, path: str):
        with open(path) as f:
            return cls.from_dict(yaml.safe_load(f) or {})


def opt(default, help: str = ""):
    if isinstance(default, (list, dict)):
        return field(default_factory=lambda: type(default)(default), metadata={"help": help})
    return field(default=default, metadata={"help": help})


# --------------------------------------------------------------------------- model
@dataclass
class PositionalEmbeddingConfig(BaseConfig):
    type: str = opt("absolute", "absolute (learned) | rope | sinusoidal | none")
    base: float = opt(10000.0, "rotary base (theta)")
    scaling_factor: float = opt(1.0, "position scaling factor for rotary embeddings")
    offset: int = opt(0, "first position index of a sequence")
    interleaved: bool = opt(True, "rotate (2i, 2i+1) pairs (native layout); False = rotate-half (HF layout)")
    rotary_fraction: Optional[float] = opt(None, "fraction of each head that is rotated (None = family default; Phi: 0.4 / 0.5)")


@dataclass
class MoEConfig(BaseConfig):
    num_experts: int = opt(0, "routed experts per MoE layer (0 = dense model)")
    top_k: int = opt(2, "experts per token")
    expert_d_ffn: int = opt(0, "hidden size of one routed expert")
    num_shared_experts: int = opt(0, "always-on experts applied to every token")
    shared_expert_d_ffn: int = opt(0, "hidden size of one shared expert (0 = expert_d_ffn)")
    shared_expert_gate: bool = opt(False, "scale the shared experts' output per token by sigmoid(x . g) (Qwen-MoE)")
    aux_loss_coeff: float = opt(0.01, "load-balance loss coefficient")
    router: str = opt("softmax_topk", "router type")
    normalize_topk: bool = opt(False, "renormalise the selected probabilities to sum to 1")
    layer_freq: int = opt(1, "every n-th layer is MoE")
    capacity_factor: float = opt(0.0, "0 = dropless")


@dataclass
class ModelConfig(BaseConfig):
    name: Optional[str] = opt(None, "model family name (gpt2, llama, gemma1, qwen, phi1, phi2, dummy, ...)")
    d_model: int = opt(512, "hidden size")
    d_ffn: int = opt(2048, "feed-forward hidden size")
    num_layers: int = opt(2, "number of transformer layers")
    num_attention_heads: Optional[int] = opt(8, "number of query heads")
    num_attention_groups: Optional[int] = opt(None, "number of key/value heads (GQA / MQA)")
    head_dim: Optional[int] = opt(None, "per-head dimension (default d_model / heads)")
    max_len: int = opt(512, "unused, kept for compatibility")
    max_position_embeddings: int = opt(512, "size of the learned position table")
    max_seq_len: int = opt(512, "training sequence length")
    dropout_embd: float = opt(0.1, "embedding dropout")
    dropout_attn: float = opt(0.1, "attention dropout")
    dropout_mlp: float = opt(0.1, "MLP dropout")
    attention_dropout: float = opt(0.1, "unused, kept for compatibility")
    attention_head_size: int = opt(64, "unused, kept for compatibility")
    precision: str = opt("bfloat16", "parameter / compute dtype")
    reset_position_ids: bool = opt(True, "restart positions after an end-of-document token")
    reset_attention_mask: bool = opt(True, "block attention across documents")
    eod_mask_loss: bool = opt(False, "leave positions whose target is the end-of-document or padding token out of the loss")
    positional_embedding: PositionalEmbeddingConfig = field(default_factory=PositionalEmbeddingConfig)
    add_pooler: bool = opt(True, "unused, kept for compatibility")
    untie_embed: bool = opt(False, "separate LM head")
    no_bias: bool = opt(False, "no bias in linear layers and norms")
    qkv_bias: Optional[bool] = opt(None, "bias on q/k/v projections only (Qwen); None = follow no_bias")
    fp32_residual_connection: bool = opt(False, "accepted for compatibility: the residual stream stays in the parameter dtype (sums inside the kernels are fp32); a warning is issued when set")
    fp16_lm_cross_entropy: bool = opt(False, "cross entropy in 16-bit")
    ln_type: str = opt("layernorm", "layernorm | rmsnorm")
    ln_eps: float = opt(1e-5, "norm epsilon")
    norm_weight_offset: Optional[float] = opt(None, "added to the norm gain (None = family default; Gemma uses 1.0)")
    post_ln: bool = opt(False, "post-LN residual topology")
    parallel_block: Optional[bool] = opt(None, "attention and MLP read the same norm output (None = family default; Phi)")
    embed_scale: Optional[float] = opt(None, "multiply embeddings (None = family default; Gemma: sqrt(d_model))")
    lm_head_bias: Optional[bool] = opt(None, "bias on the LM head (None = family default; Phi)")
    lm_head_chunk: int = opt(0, "vocabulary columns per step of the chunked LM head + cross entropy (multiple of "
                                "128; 0 = materialise the logits, chunked by itself without gradients above 64 k)")
    activation_type: str = opt("gelu", "relu|gelu|gelu_tanh|silu|swiglu|geglu|reglu|glu")
    seq_len_q: Optional[int] = opt(None, "unused")
    seq_len_kv: Optional[int] = opt(None, "unused")
    moe: MoEConfig = field(default_factory=MoEConfig)
    hf_model_type: Optional[str] = opt(None, "HuggingFace model_type")
    hf_architecture: Optional[str] = opt(None, "HuggingFace architecture name")
    tokenizer_type: str = opt("gpt2", "tokenizer type")
    vocab_name_or_path: str = opt("gpt2", "vocab name or path")
    merge_file_path: Optional[str] = opt(None, "merge file path")
    vocab_size: Optional[int] = opt(None, "set by the tokenizer (or directly for synthetic data)")
    padded_vocab_size: Optional[int] = opt(None, "vocab padded to vocab_padding_unit * tp")
    eod_token_id: Optional[int] = opt(None, "end-of-document id (set by the tokenizer)")
    pad_token_id: Optional[int] = opt(None, "padding id (set by the tokenizer)")

    def __post_init__(self):
        if self.ln_type not in ("layernorm", "rmsnorm"):
            raise ValueError(f"Invalid layer norm type: {self.ln_type}")


# --------------------------------------------------------------------------- trainer / operation / init
@dataclass
class TrainerConfig(BaseConfig):
    model_name: str = opt("model", "run name")
    config_path: Optional[str] = opt(None, "config file path")
    model_path: str = opt("", "checkpoint directory")
    init_from_hf: Optional[str] = opt(None, "HuggingFace checkpoint directory to initialise the weights from when "
                                            "model_path holds no checkpoint to resume (fine-tuning)")
    micro_batch_size: Optional[int] = opt(2, "micro batch size")
    train_batch_size: Optional[int] = opt(None, "global batch size")
    gradient_accumulation_steps: Optional[int] = opt(None, "gradient accumulation steps")
    do_eval: bool = opt(False, "run evaluation")
    eval_batch_size: Optional[int] = opt(None, "eval batch size")
    do_eval_subtask: bool = opt(False, "run evaluation subtasks")
    test_batch_size: Optional[int] = opt(None, "test batch size")
    do_test: bool = opt(False, "run test at the end")
    save_checkpoint_steps: int = opt(1000, "checkpoint cadence")
    log_interval: int = opt(20, "log cadence")
    grad_norm_log_interval: Optional[Literal["log", "checkpoint"]] = opt(None, "None | log | checkpoint")
    param_norm_log_interval: Optional[Literal["log", "checkpoint"]] = opt(None, "None | log | checkpoint")
    num_workers: int = opt(8, "dataset workers")
    tensor_model_parallel_size: int = opt(1, "tensor parallel size")
    pipeline_model_parallel_size: int = opt(1, "pipeline parallel size (must be 1)")
    vocab_padding_unit: int = opt(128, "vocab padding unit")
    special_tokens_config_path: Optional[str] = opt(None, "JSON / YAML file of special tokens (eos_token, pad_token, eod_token, *_token_id), looked up under model.vocab_name_or_path, then trainer.model_path")
    use_flash_attn: bool = opt(True, "fused attention kernel")
    cuda_graph: bool = opt(False, "capture one micro-batch forward+backward in a CUDA graph and replay it")
    compile_model: bool = opt(False, "accepted for compatibility; the hot path is hand-written kernels")
    compile_mode: Optional[Literal["default", "reduce-overhead", "max-autotune"]] = opt("default", "ignored")
    compile_backend: Literal["inductor", "cudagraphs", "eager"] = opt("inductor", "ignored")
    compile_dynamic: bool = opt(False, "ignored")
    compile_fullgraph: bool = opt(False, "ignored")


@dataclass
class OperationConfig(BaseConfig):
    train_steps: int = opt(1000, "train steps")
    eval_interval: int = opt(100, "evaluation interval")
    eval_samples: int = opt(100, "evaluation sample count")
    test_samples: int = opt(100, "test sample count")
    activation_recompute: bool = opt(False, "recompute layer activations in backward")
    recompute_strategy: Optional[str] = opt("default", "default | optimized")
    no_save: bool = opt(False, "never write checkpoints")
    resume_data_position: bool = opt(True, "after a resume, continue the training data stream where the checkpoint "
                                           "left it (skips the micro-batches of the completed steps) instead of "
                                           "replaying it from the start")
    exit_interval: Optional[int] = opt(None, "stop after this many steps")
    save_dist_ckpt: bool = opt(False, "one checkpoint shard per TP rank")


@dataclass
class InitConfig(BaseConfig):
    seed: int = opt(1337, "random seed")
    data_parallel_random_init: bool = opt(False, "different init per DP rank")
    init_std: float = opt(0.006, "normal init std")
    xavier_init: Optional[bool] = opt(False, "xavier uniform init")


# --------------------------------------------------------------------------- optim
@dataclass
class OptimConfig(BaseConfig):
    optimizer: str = opt("adam", "adam | muon")
    lr_scheduler: str = opt("cosine", "cosine | linear | constant")
    max_lr: float = opt(5e-4, "peak learning rate")
    min_lr: float = opt(0.0, "final learning rate")
    warmup_steps: int = opt(0, "linear warm-up steps")
    annealing_steps: int = opt(0, "decay steps (0 = train_steps)")
    weight_decay: float = opt(0.01, "decoupled weight decay")
    no_decay_on_embedding: bool = opt(True, "no decay on learned position tables")
    adam_eps: float = opt(1e-8, "adam epsilon")
    adam_beta1: float = opt(0.9, "adam beta1")
    adam_beta2: float = opt(0.95, "adam beta2")
    clip_grad: float = opt(1.0, "global grad-norm clip (0 = off)")
    load_checkpoint_optim_state: bool = opt(True, "restore optimizer state on resume")
    load_checkpoint_lr_scheduler: bool = opt(True, "restore scheduler state on resume")
    muon_lr: float = opt(0.02, "Muon learning rate for 2-D hidden matrices")
    muon_momentum: float = opt(0.95, "Muon momentum")
    muon_ns_steps: int = opt(5, "Newton-Schulz iterations")
    nesterov: bool = opt(True, "Nesterov momentum in Muon")
    muon_weight_decay: float = opt(0.0, "decoupled decay on Muon parameters")
    cpu_offload_optimizer: bool = opt(False, "keep Adam moments in pinned host memory")
    master_weights: bool = opt(False, "fp32 master copy of 16-bit parameters")
    fp32_grad_accum: bool = opt(True, "accumulate gradients in an fp32 buffer (False = parameter dtype)")


# --------------------------------------------------------------------------- parallel
@dataclass
class ParallelConfig(BaseConfig):
    rank: int = opt(-1, "global rank")
    local_rank: int = opt(0, "local rank")
    world_size: int = opt(1, "world size")
    dist_backend: str = opt("nccl", "nccl on CUDA, gloo on CPU")
    timeout_minute: float = opt(10.0, "process-group timeout in minutes")
    sequence_parallel: bool = opt(False, "Megatron sequence parallelism inside the TP group")
    expert_model_parallel_size: int = opt(1, "expert parallel size")
    zero_stage: int = opt(0, "0 = replicated optimizer, 1 = optimizer state sharded over DP")
    fused_comm: bool = opt(True, "use the in-kernel P2P collectives when symmetric memory is available")
    fused_norm_gather: Literal["auto", "on", "off"] = opt(
        "auto", "row-parallel GEMM -> reduce-scatter -> RMSNorm -> all-gather in one kernel (auto: separate kernels)")
    fused_zero: bool = opt(True, "gradient reduce-scatter + Adam + parameter broadcast as in-kernel collectives")
    fused_moe: bool = opt(True, "expert-parallel dispatch / combine as in-kernel P2P copies")
    nvls: Literal["auto", "on", "off"] = opt("auto", "NVSwitch multicast (multimem) forms of the in-kernel collectives")
    grad_bucket_mb: float = opt(64.0, "gradient reduction bucket size in MiB (overlap_grad_reduce)")
    overlap_grad_reduce: bool = opt(False, "reduce gradient buckets over the data-parallel group while the last "
                                           "micro-batch's backward pass still runs (instead of one reduction of "
                                           "the whole buffer inside the optimizer step)")
    use_fsdp: bool = opt(False, "fully sharded data parallel")
    fsdp_fused_gather: bool = opt(False, "FSDP parameter gathers as P2P / NVSwitch-multicast kernels into "
                                         "symmetric slots instead of NCCL all-gathers")
    fsdp_offload_params: bool = opt(False, "keep FSDP shards in pinned host memory")
    fsdp_mixed_precision: Literal["fp16", "float16", "bf16", "bfloat16", "fp32", "float32", "mixed"] = opt(
        "mixed", "FSDP reduce precision")
    fsdp_sharding_strategy: Literal["full", "hybrid", "no_shard"] = opt("full", "FSDP sharding strategy")
    fsdp_state_dict_type: Literal["full", "local", "sharded"] = opt("full", "FSDP state-dict type")


# --------------------------------------------------------------------------- utils
@dataclass
class UtilsConfig(BaseConfig):
    log_level: str = opt("INFO", "log level")
    profile_nsys: bool = opt(False, "bracket steps with cudaProfilerStart/Stop")
    profile_torch: bool = opt(False, "torch profiler trace")
    profile_step_start: Optional[int] = opt(10, "first profiled step")
    profile_step_end: Optional[int] = opt(12, "last profiled step")
    profile_ranks: Optional[List[int]] = opt([0], "ranks that profile")
    stop_on_profile_end: bool = opt(False, "accepted for compatibility: training always stops when a profiling window ends, as in the reference")
    deterministic: bool = opt(False, "deterministic algorithms")
    report_memory_usage: bool = opt(True, "memory report at the first log step")
    tensorboard_dir: Optional[str] = opt(None, "tensorboard directory")
    mlflow_tracking_uri: Optional[str] = opt(None, "mlflow tracking uri")
    mlflow_experiment_name: Optional[str] = opt(None, "mlflow experiment")
    heartbeat_interval_s: float = opt(0.0, "host-side rank heartbeat period (0 = off)")
    heartbeat_timeout_s: float = opt(60.0, "declare a rank dead after this silence")


# --------------------------------------------------------------------------- data
@dataclass
class DataConfig(BaseConfig):
    """Free-form group: unknown keys are stored as attributes (the data YAML owns its schema)."""

    task_type: str = opt("pretrain", "pretrain | sft | dpo | synthetic")
    config_path: Optional[str] = opt(None, "dataset YAML (UniversalDataConfig)")
    data_path: Optional[List[Union[float, str]]] = opt(None, "legacy weighted data paths")
    splits: List[float] = opt([0.97, 0.029, 0.001], "train/eval/test ratios")
    train_datasets: Optional[List[Union[float, str]]] = opt(None, "train datasets")
    eval_datasets: Optional[List[Union[float, str]]] = opt(None, "eval datasets")
    test_datasets: Optional[List[Union[float, str]]] = opt(None, "test datasets")
    vocab_size: int = opt(51200, "vocab size")
    num_token_types: int = opt(2, "token types")
    pad_to_max_length: bool = opt(False, "pad samples to max length")
    pad_token_id: int = opt(-1, "PAD id (-1 = EOS)")
    synthetic_seed: int = opt(1234, "seed of the synthetic uniform-token stream")

    def update(self, **kwargs):
        known = {f.name for f in fields(self)}
        extra = {k: v for k, v in kwargs.items() if k not in known}
        BaseConfig.update(self, **{k: v for k, v in kwargs.items() if k in known})
        for k, v in extra.items():
            setattr(self, k, v)
        return self


# --------------------------------------------------------------------------- rl
@dataclass
class RLConfig(BaseConfig):
    algorithm: str = opt("grpo", "grpo (rollouts + clipped policy gradient); preference pairs train with data.task_type: dpo")
    num_prompts: int = opt(64, "prompts per rollout batch")
    prompt_len: int = opt(256, "synthetic prompt length")
    group_size: int = opt(8, "samples per prompt")
    max_new_tokens: int = opt(512, "generated tokens per sample")
    temperature: float = opt(1.0, "sampling temperature")
    top_p: float = opt(1.0, "nucleus sampling threshold")
    top_k: int = opt(0, "top-k sampling (0 = off)")
    clip_eps: float = opt(0.2, "PPO clip epsilon")
    kl_beta: float = opt(0.04, "KL penalty to the frozen reference policy")
    kv_block_size: int = opt(16, "tokens per KV-cache page")
    reward_vocab_subset: int = opt(1024, "size of the seeded rewarded-token subset")
    reward_seed: int = opt(7, "seed of the rewarded subset / prompts")
    adv_eps: float = opt(1e-6, "epsilon in the group advantage normalisation")
    dpo_beta: float = opt(0.1, "DPO: scale of the policy / reference log-ratio difference (data.task_type: dpo)")
    dpo_label_smoothing: float = opt(0.0, "DPO: weight of the flipped pair's loss (conservative DPO)")


@dataclass
class MainConfig(BaseConfig):
    model: ModelConfig = field(default_factory=ModelConfig)
    init: InitConfig = field(default_factory=InitConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    data: DataConfig = field(default_factory=DataConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    operation: OperationConfig = field(default_factory=OperationConfig)
    utils: UtilsConfig = field(default_factory=UtilsConfig)
    rl: RLConfig = field(default_factory=RLConfig)


GROUPS = ("model", "init", "optim", "data", "parallel", "trainer", "operation", "utils", "rl")
