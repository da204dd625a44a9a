"""HuggingFace interop must be forward-equivalent: logits of a tiny random `transformers` model and of
the native model loaded from it agree, and an exported native model reloads into `transformers`."""

import pytest
import torch

from helpers import tiny_config

transformers = pytest.importorskip("transformers")


def _native(family, **kw):
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    cfg = tiny_config(family, **kw)
    validate_config(cfg)
    return cfg, LanguageModel(cfg).eval()


def test_architecture_aliases():
    from ironcore_b200.checkpoint.hf_interop import Architecture, detect_architecture

    assert detect_architecture("gpt2") == Architecture.GPT2
    assert detect_architecture("gpt2-small") == Architecture.GPT2
    for name in ("llama", "llama3", "mistral", "qwen2", "gemma", "something-new"):
        assert detect_architecture(name) == Architecture.LLAMA
    for name in ("phi", "phi-2", "phi1"):
        assert detect_architecture(name) == Architecture.PHI


def test_gpt2_forward_equivalence_and_roundtrip(tmp_path):
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface, load_from_huggingface

    torch.manual_seed(0)
    hcfg = transformers.GPT2Config(vocab_size=512, n_positions=32, n_embd=64, n_layer=2, n_head=4, n_inner=128,
                                   resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, activation_function="gelu")
    hf = transformers.GPT2LMHeadModel(hcfg).eval()
    cfg, model = _native("gpt2", hf_model_type="gpt2")
    load_from_huggingface(model, cfg, {k: v for k, v in hf.state_dict().items()})
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        ref = hf(ids).logits
        got = model(ids)[..., :512]
    assert torch.allclose(ref, got, atol=2e-4), (ref - got).abs().max()
    out = export_to_huggingface(model, cfg, tmp_path / "hf_gpt2")
    back = transformers.GPT2LMHeadModel.from_pretrained(out).eval()
    with torch.no_grad():
        again = back(ids).logits
    assert torch.allclose(ref, again, atol=2e-4)


@pytest.mark.parametrize("interleaved", [True, False])
def test_llama_forward_equivalence_and_roundtrip(tmp_path, interleaved):
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface, load_from_huggingface, read_hf_state_dict

    torch.manual_seed(1)
    hcfg = transformers.LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                    rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                                    attention_bias=False)
    hf = transformers.LlamaForCausalLM(hcfg).eval()
    cfg, model = _native("llama", hf_model_type="llama",
                         positional_embedding={"type": "rope", "base": 10000.0, "interleaved": interleaved})
    load_from_huggingface(model, cfg, {k: v for k, v in hf.state_dict().items()})
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        ref = hf(ids).logits
        got = model(ids)[..., :512]
    assert torch.allclose(ref, got, atol=3e-4), (ref - got).abs().max()
    out = export_to_huggingface(model, cfg, tmp_path / "hf_llama", max_shard_bytes=100_000)
    assert (out / "model.safetensors.index.json").exists()
    sd = read_hf_state_dict(out)
    for k, v in hf.state_dict().items():
        assert torch.allclose(v, sd[k], atol=1e-6), k


def _logits_match(hf, model, cfg, vocab=512, atol=3e-4):
    from ironcore_b200.checkpoint.hf_interop import load_from_huggingface

    load_from_huggingface(model, cfg, dict(hf.state_dict()))
    ids = torch.randint(0, vocab, (2, 32))
    with torch.no_grad():
        ref, got = hf(ids).logits, model(ids)[..., :vocab]
    assert torch.allclose(ref, got, atol=atol), (ref - got).abs().max()
    return ids, ref


def _export_reloads(model, cfg, hf_cls, out_dir, ids, ref):
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface

    back = hf_cls.from_pretrained(export_to_huggingface(model, cfg, out_dir)).eval()
    with torch.no_grad():
        assert torch.allclose(ref, back(ids).logits, atol=2e-4), (ref - back(ids).logits).abs().max()


def test_qwen2_forward_equivalence_and_roundtrip(tmp_path):
    """Qwen family: biases on q / k / v only, RMSNorm eps 1e-6, rotary base 1e6, grouped keys / values."""
    torch.manual_seed(2)
    hcfg = transformers.Qwen2Config(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                    rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    hf = transformers.Qwen2ForCausalLM(hcfg).eval()
    cfg, model = _native("qwen", hf_model_type="qwen2", ln_eps=1e-6, positional_embedding={"type": "rope", "base": 1e6})
    assert cfg.model.qkv_bias and model.model.layers[0].attn_output.bias is None
    ids, ref = _logits_match(hf, model, cfg)
    _export_reloads(model, cfg, transformers.Qwen2ForCausalLM, tmp_path / "hf_qwen2", ids, ref)


def test_gemma_forward_equivalence_and_roundtrip(tmp_path):
    """Gemma-1 family: (1 + w) norm gains, sqrt(d) embedding scale, GeGLU, one key / value head, tied head."""
    torch.manual_seed(3)
    hcfg = transformers.GemmaConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=1, head_dim=16,
                                    max_position_embeddings=32, rms_norm_eps=1e-6, rope_theta=10000.0,
                                    hidden_act="gelu_pytorch_tanh", hidden_activation="gelu_pytorch_tanh")
    hf = transformers.GemmaForCausalLM(hcfg).eval()
    cfg, model = _native("gemma1", hf_model_type="gemma", ln_eps=1e-6, no_bias=True, ln_type="rmsnorm",
                         num_attention_groups=1, activation_type="geglu", untie_embed=False,
                         positional_embedding={"type": "rope", "base": 10000.0})
    assert cfg.model.norm_weight_offset == 1.0 and cfg.model.embed_scale == 8.0
    ids, ref = _logits_match(hf, model, cfg)
    _export_reloads(model, cfg, transformers.GemmaForCausalLM, tmp_path / "hf_gemma", ids, ref)


@pytest.mark.parametrize("interleaved", [True, False])
def test_phi_forward_equivalence_and_roundtrip(tmp_path, interleaved):
    """Phi family: attention and MLP in parallel behind one LayerNorm, rotary on half of every head, biases
    everywhere including the LM head; export reloads into ``transformers``."""
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface

    torch.manual_seed(4)
    hcfg = transformers.PhiConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                  num_attention_heads=4, max_position_embeddings=32, layer_norm_eps=1e-5,
                                  rope_theta=10000.0, partial_rotary_factor=0.5, hidden_act="gelu_new",
                                  resid_pdrop=0.0, embd_pdrop=0.0, attention_dropout=0.0)
    hf = transformers.PhiForCausalLM(hcfg).eval()
    cfg, model = _native("phi2", hf_model_type="phi", ln_eps=1e-5, activation_type="gelu_new", untie_embed=True,
                         positional_embedding={"type": "rope", "base": 10000.0, "rotary_fraction": 0.5,
                                               "interleaved": interleaved})
    assert cfg.model.parallel_block and cfg.model.lm_head_bias
    ids, ref = _logits_match(hf, model, cfg)
    out = export_to_huggingface(model, cfg, tmp_path / "hf_phi")
    back = transformers.PhiForCausalLM.from_pretrained(out).eval()
    with torch.no_grad():
        assert torch.allclose(ref, back(ids).logits, atol=2e-4)


def test_mixtral_forward_equivalence_and_roundtrip(tmp_path):
    """Mixture of experts in the Mixtral layout (every layer: softmax router, top-2 renormalised, SwiGLU experts, no
    shared expert): the native block reproduces ``transformers``' logits, and the export (per-expert names, as
    checkpoints on disk carry them) reloads into ``transformers``."""
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    torch.manual_seed(5)
    hcfg = transformers.MixtralConfig(vocab_size=512, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, num_local_experts=4, num_experts_per_tok=2,
                                      sliding_window=None, tie_word_embeddings=False, router_aux_loss_coef=0.0)
    hf = transformers.MixtralForCausalLM(hcfg).eval()
    mesh.destroy_model_parallel()
    cfg = tiny_config("llama", d_ffn=96, hf_model_type="mixtral", ln_eps=1e-5,
                      positional_embedding={"type": "rope", "base": 10000.0})
    cfg.model.moe(num_experts=4, top_k=2, expert_d_ffn=96, normalize_topk=True, aux_loss_coeff=0.0)
    validate_config(cfg)
    model = LanguageModel(cfg).eval()
    ids, ref = _logits_match(hf, model, cfg)
    out = export_to_huggingface(model, cfg, tmp_path / "hf_mixtral")
    back = transformers.MixtralForCausalLM.from_pretrained(out).eval()
    with torch.no_grad():
        assert torch.allclose(ref, back(ids).logits, atol=2e-4)


def test_qwen2_moe_forward_equivalence_and_roundtrip(tmp_path):
    """Routed experts plus an always-on shared expert (the Qwen-MoE layout: top-k of the softmax without
    renormalisation, the shared expert scaled by a sigmoid gate): native logits equal ``transformers``', and the
    export reloads into ``transformers``."""
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    torch.manual_seed(6)
    hcfg = transformers.Qwen2MoeConfig(vocab_size=512, hidden_size=64, intermediate_size=128, moe_intermediate_size=48,
                                       shared_expert_intermediate_size=80, num_hidden_layers=2, num_attention_heads=4,
                                       num_key_value_heads=2, max_position_embeddings=32, rms_norm_eps=1e-6,
                                       rope_theta=1e6, num_experts=8, num_experts_per_tok=3, norm_topk_prob=False,
                                       decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False,
                                       router_aux_loss_coef=0.0, use_sliding_window=False)
    hf = transformers.Qwen2MoeForCausalLM(hcfg).eval()
    mesh.destroy_model_parallel()
    cfg = tiny_config("qwen", hf_model_type="qwen2_moe", ln_eps=1e-6, positional_embedding={"type": "rope", "base": 1e6})
    cfg.model.moe(num_experts=8, top_k=3, expert_d_ffn=48, num_shared_experts=1, shared_expert_d_ffn=80,
                  shared_expert_gate=True, normalize_topk=False, aux_loss_coeff=0.0)
    validate_config(cfg)
    model = LanguageModel(cfg).eval()
    ids, ref = _logits_match(hf, model, cfg)
    out = export_to_huggingface(model, cfg, tmp_path / "hf_qwen2_moe")
    back = transformers.Qwen2MoeForCausalLM.from_pretrained(out).eval()
    with torch.no_grad():
        assert torch.allclose(ref, back(ids).logits, atol=2e-4)


def _tp_import_worker(rank, world, path):
    import torch.distributed as dist

    from ironcore_b200.checkpoint.hf_interop import load_from_huggingface
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    saved = torch.load(path)
    cfg = tiny_config("qwen", hf_model_type="qwen2", ln_eps=1e-6, positional_embedding={"type": "rope", "base": 1e6})
    cfg.trainer(tensor_model_parallel_size=world)
    cfg.parallel(world_size=world, rank=rank, sequence_parallel=True)
    validate_config(cfg)
    mesh.initialize_model_parallel(world, sequence_parallel=True)
    model = LanguageModel(cfg).eval()
    load_from_huggingface(model, cfg, saved["sd"])
    with torch.no_grad():
        local = model(saved["ids"])                                   # [B, S, V / world]
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous())
    full = torch.cat(parts, dim=-1)[..., :512]
    assert torch.allclose(full, saved["logits"], atol=3e-4), (full - saved["logits"]).abs().max()


def test_import_into_two_tensor_parallel_ranks_matches_transformers(tmp_path):
    """The HuggingFace import splits q | k | v, gate | up, the row-parallel projections and the vocabulary over the
    tensor-parallel group (with sequence parallelism on): the gathered logits equal ``transformers``'."""
    from helpers import run_distributed

    torch.manual_seed(7)
    hcfg = transformers.Qwen2Config(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                    rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    hf = transformers.Qwen2ForCausalLM(hcfg).eval()
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        logits = hf(ids).logits
    path = str(tmp_path / "hf.pt")
    torch.save({"sd": {k: v.clone() for k, v in hf.state_dict().items()}, "ids": ids, "logits": logits}, path)
    run_distributed(_tp_import_worker, 2, path)


def _ep_import_worker(rank, world, path):
    from ironcore_b200.checkpoint.hf_interop import load_from_huggingface
    from ironcore_b200.config import validate_config
    from ironcore_b200.models import LanguageModel
    from ironcore_b200.parallel import mesh

    saved = torch.load(path)
    cfg = tiny_config("llama", d_ffn=96, hf_model_type="mixtral", ln_eps=1e-5,
                      positional_embedding={"type": "rope", "base": 10000.0})
    cfg.model.moe(num_experts=4, top_k=2, expert_d_ffn=96, normalize_topk=True, aux_loss_coeff=0.0)
    cfg.trainer(micro_batch_size=2, train_batch_size=4, gradient_accumulation_steps=None)
    cfg.parallel(world_size=world, rank=rank, expert_model_parallel_size=world)
    validate_config(cfg)
    mesh.initialize_model_parallel(1, expert_model_parallel_size=world)
    model = LanguageModel(cfg).eval()
    assert model.model.layers[0].mlp.experts_up.shape[0] == 4 // world
    load_from_huggingface(model, cfg, saved["sd"])
    with torch.no_grad():
        got = model(saved["ids"])[..., :512]
    assert torch.allclose(got, saved["logits"], atol=3e-4), (got - saved["logits"]).abs().max()
    # the export gathers the experts of both ranks again (collective; rank 0 writes)
    from ironcore_b200.checkpoint.hf_interop import export_to_huggingface, read_hf_state_dict

    out = export_to_huggingface(model, cfg, saved["out_dir"])
    import torch.distributed as dist

    dist.barrier()
    if rank == 0:
        back = read_hf_state_dict(out)
        w1 = back["model.layers.1.block_sparse_moe.experts.3.w1.weight"]
        assert torch.allclose(w1, saved["sd"]["model.layers.1.mlp.experts.gate_up_proj"][3, :96], atol=1e-6)


def test_import_of_a_mixture_of_experts_over_two_expert_parallel_ranks(tmp_path):
    """Each expert-parallel rank keeps its experts of a Mixtral checkpoint; with the token exchange between the
    ranks the logits equal ``transformers``'."""
    from helpers import run_distributed

    torch.manual_seed(8)
    hcfg = transformers.MixtralConfig(vocab_size=512, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, num_local_experts=4, num_experts_per_tok=2,
                                      sliding_window=None, tie_word_embeddings=False, router_aux_loss_coef=0.0)
    hf = transformers.MixtralForCausalLM(hcfg).eval()
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        logits = hf(ids).logits
    path = str(tmp_path / "hf.pt")
    torch.save({"sd": {k: v.clone() for k, v in hf.state_dict().items()}, "ids": ids, "logits": logits,
                "out_dir": str(tmp_path / "hf_out")}, path)
    run_distributed(_ep_import_worker, 2, path)
    back = transformers.MixtralForCausalLM.from_pretrained(tmp_path / "hf_out").eval()
    with torch.no_grad():
        assert torch.allclose(back(ids).logits, logits, atol=2e-4)


def test_trainer_starts_from_a_huggingface_checkpoint(tmp_path):
    """``trainer.init_from_hf``: without a checkpoint to resume, training starts from the HuggingFace weights (through
    the flat parameter buffer of the optimizer engine); with one, the resume wins."""
    from ironcore_b200.checkpoint import save_checkpoint
    from ironcore_b200.config import validate_config
    from ironcore_b200.parallel import mesh
    from ironcore_b200.trainer import Trainer

    torch.manual_seed(9)
    hcfg = transformers.LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                    rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hcfg).eval()
    hf.save_pretrained(tmp_path / "hf", safe_serialization=True)
    ids = torch.randint(0, 512, (2, 32))
    with torch.no_grad():
        ref = hf(ids).logits

    def trainer():
        mesh.destroy_model_parallel()
        cfg = tiny_config("llama", hf_model_type="llama")
        cfg.trainer(init_from_hf=str(tmp_path / "hf"), model_path=str(tmp_path / "ck"))
        validate_config(cfg)
        return cfg, Trainer(cfg)

    cfg, tr = trainer()
    assert tr.load_or_init_weights() == 0
    tr.model.eval()
    with torch.no_grad():
        assert torch.allclose(tr.model(ids)[..., :512], ref, atol=3e-4)
    tr.model.train()
    tr.train_step(0)                                       # the optimizer engine updates the loaded weights
    save_checkpoint(cfg, tr.model, tr.optimizer, tr.lr_scheduler, 0)
    after = {k: v.clone() for k, v in tr.model.canonical_state_dict().items()}
    cfg2, tr2 = trainer()
    assert tr2.load_or_init_weights() == 1                 # resumes the native checkpoint, not the HuggingFace one
    for k, v in tr2.model.canonical_state_dict().items():
        assert torch.equal(v, after[k]), k


def test_export_subcommand_writes_a_loadable_directory(tmp_path, capsys):
    """``ironcore train`` then ``ironcore export``: the written directory loads into ``transformers`` and holds the
    trained weights."""
    import yaml

    from ironcore_b200.__main__ import main
    from ironcore_b200.checkpoint.hf_interop import read_hf_state_dict
    from ironcore_b200.parallel import mesh

    mesh.destroy_model_parallel()
    run = {"trainer": {"micro_batch_size": 2, "train_batch_size": 2, "log_interval": 1, "save_checkpoint_steps": 2,
                       "model_path": str(tmp_path / "ck"), "use_flash_attn": False, "vocab_padding_unit": 8},
           "operation": {"train_steps": 2},
           "model": {"name": "llama", "hf_model_type": "llama", "d_model": 32, "d_ffn": 64, "num_layers": 2,
                     "num_attention_heads": 4, "num_attention_groups": 2, "max_seq_len": 32,
                     "max_position_embeddings": 32, "precision": "fp32", "ln_type": "rmsnorm",
                     "activation_type": "swiglu", "no_bias": True, "untie_embed": True, "vocab_size": 300,
                     "dropout_embd": 0.0, "dropout_attn": 0.0, "dropout_mlp": 0.0,
                     "positional_embedding": {"type": "rope"}},
           "data": {"task_type": "synthetic", "vocab_size": 300}, "optim": {"max_lr": 1e-3, "warmup_steps": 0}}
    path = tmp_path / "run.yaml"
    path.write_text(yaml.safe_dump(run))
    assert main(["train", "--config", str(path)]) == 0
    mesh.destroy_model_parallel()
    assert main(["export", "--config", str(path), "--output", str(tmp_path / "hf")]) == 0
    assert "exported step 1" in capsys.readouterr().out
    back = transformers.LlamaForCausalLM.from_pretrained(tmp_path / "hf").eval()
    sd = read_hf_state_dict(tmp_path / "hf")
    assert back.config.num_key_value_heads == 2 and sd["model.embed_tokens.weight"].shape[1] == 32
    with torch.no_grad():
        assert torch.isfinite(back(torch.randint(0, 300, (1, 8))).logits).all()
    mesh.destroy_model_parallel()
