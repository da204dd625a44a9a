"""Causal language model: embedding -> transformer stack -> final norm -> LM head ->
vocab-parallel cross entropy -> masked mean.

``forward(input_ids, labels=None, ...)`` returns the scalar loss when labels are given and
the (vocab-sharded) logits ``[B, S, V/t]`` otherwise. Document boundaries (positions and
attention restarting after an end-of-document token) are derived on the device and passed
to the attention kernel as ``cu_seqlens`` — no ``[B,1,S,S]`` mask is ever built on the
fused path. Labels equal to ``-100`` are excluded from the loss.
(Behavioural reference: ironcore/language_model.py:21-234; parameter names follow the
reference's live model so checkpoints interoperate: ironcore/models/transformer.py:47-72.)
"""

from __future__ import annotations

import math
from collections import OrderedDict
from typing import Callable, Dict, Optional

import torch

from ..layers.embedding import LanguageModelEmbedding
from ..layers.module import BaseModule, init_parameters
from ..layers.norm import get_norm
from ..ops import functional as OF
from ..parallel import collectives as C
from ..parallel import mesh
from ..parallel.tensor_parallel import ColumnParallelLinear, vocab_parallel_cross_entropy
from .families import resolve_family_defaults

IGNORE_INDEX = -100

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
           "half": torch.float16, "float32": torch.float32, "fp32": torch.float32, "float": torch.float32}


def get_model_dtype(config) -> torch.dtype:
    try:
        return _DTYPES[str(config.model.precision).lower()]
    except KeyError as exc:
        raise ValueError(f"unknown precision {config.model.precision}") from exc


def masked_mean_loss(per_token_loss: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
    """sum(loss * mask) / sum(mask) (reference: ironcore/training_utils.py:142-151)."""
    mask = loss_mask.reshape(-1).float()
    return (per_token_loss.reshape(-1).float() * mask).sum() / mask.sum().clamp_min(1.0)


class _LinearT(torch.autograd.Function):
    """y = x @ W^T for a weight stored [out, in] (the tied LM head reads the embedding table)."""

    @staticmethod
    def forward(ctx, x, weight):
        from ..ops import kernels

        ctx.save_for_backward(x, weight)
        return kernels.mm_nt(x, weight)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import kernels

        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = kernels.mm_nn(dy, weight) if ctx.needs_input_grad[0] else None
        dw = kernels.mm_tn(dy, x) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear_t(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if OF.use_native(x):
        return _LinearT.apply(x.contiguous(), weight)
    return x @ weight.t()


class LanguageModel(BaseModule):
    def __init__(self, config, loss_fn: Optional[Callable] = None, device=None):
        super().__init__(config)
        m = config.model
        self.family = resolve_family_defaults(m)
        self.loss_fn = loss_fn or masked_mean_loss
        dtype = get_model_dtype(config)
        self.vocab_size = int(m.vocab_size if m.vocab_size is not None else config.data.vocab_size)
        tp = mesh.get_tensor_model_parallel_world_size()
        unit = config.trainer.vocab_padding_unit * tp
        self.padded_vocab_size = int(m.padded_vocab_size or (math.ceil(self.vocab_size / unit) * unit))
        m.vocab_size, m.padded_vocab_size = self.vocab_size, self.padded_vocab_size
        self.tp_group = mesh.get_tensor_model_parallel_group()
        self.tp_size = tp
        self.sequence_parallel = mesh.sequence_parallel_enabled()
        self.seq_len = m.max_seq_len
        learned_pos = m.positional_embedding.type.lower() == "absolute"
        if self.family == "DUMMY":
            from .dummy import DummyModel

            self.embedding = LanguageModelEmbedding(self.padded_vocab_size, self.vocab_size, m.d_model, m.max_seq_len,
                                                    False, 0.0, None, dtype, device)
            self.model = DummyModel(config, dtype, device)
        else:
            from .transformer import TransformerModel

            self.embedding = LanguageModelEmbedding(self.padded_vocab_size, self.vocab_size, m.d_model,
                                                    max(m.max_seq_len, 1), learned_pos, m.dropout_embd, m.embed_scale,
                                                    dtype, device)
            self.model = TransformerModel(config, dtype, device)
        self.output_layernorm = get_norm(config, dtype, device)
        self.untied = bool(m.untie_embed)
        if self.untied:
            self.output_layer = ColumnParallelLinear(m.d_model, self.padded_vocab_size, bias=bool(m.lm_head_bias),
                                                     dtype=dtype, device=device)
        self.reset_position_ids = m.reset_position_ids
        self.reset_attention_mask = m.reset_attention_mask
        self.eod_mask_loss = m.eod_mask_loss
        self.init_weights()

    # ------------------------------------------------------------------ initialisation
    def init_weights(self):
        """normal(0, init_std); residual projections (attn_output, down_proj) use
        std / sqrt(2 * num_layers); biases zero; norm gains one (or 1 - offset); padded
        vocabulary rows zero. Sharded weights are slices of the TP=1 tensor, drawn from a
        CPU generator so every TP size sees the same full matrices.
        (Behavioural reference: ironcore/layers/module.py:43-163.)"""
        # (dim, real vocabulary size) of the tensors that carry vocabulary padding: their padding is not drawn
        self.embedding.word_embeddings.weight.vocab_valid = (0, self.vocab_size)
        if self.untied:
            self.output_layer.weight.vocab_valid = (1, self.vocab_size)
        init_parameters(self, self.config)
        tp_rank = mesh.get_tensor_model_parallel_rank()
        # zero the padded vocabulary rows / columns
        with torch.no_grad():
            w = self.embedding.word_embeddings
            lo = max(self.vocab_size - w.vocab_start, 0)
            if lo < w.rows_per_partition:
                w.weight[lo:].zero_()
            if self.untied:
                v_local = self.output_layer.out_per_partition
                start = tp_rank * v_local
                lo = max(self.vocab_size - start, 0)
                if lo < v_local:
                    self.output_layer.weight[:, lo:].zero_()

    # ------------------------------------------------------------------ helpers
    def _document_layout(self, input_ids: torch.Tensor):
        """Positions restarting after every end-of-document token and the cumulative
        document boundaries of the flat token stream (int32, includes batch-row ends)."""
        eod = self.config.model.eod_token_id
        b, s = input_ids.shape
        if eod is None or not (self.reset_position_ids or self.reset_attention_mask):
            return None, None
        is_eod = input_ids == eod
        pos_ids = None
        if self.reset_position_ids:
            idx = torch.arange(s, device=input_ids.device).expand(b, s)
            # a new document starts *after* an EOD token
            start = torch.where(is_eod, idx + 1, torch.zeros_like(idx))
            start = torch.cummax(torch.roll(start, 1, dims=1).index_fill_(
                1, torch.zeros(1, dtype=torch.long, device=input_ids.device), 0), dim=1).values
            pos_ids = idx - start
        cu = None
        if self.reset_attention_mask:
            flat_end = is_eod.clone()
            flat_end[:, -1] = True
            ends = torch.nonzero(flat_end.reshape(-1), as_tuple=False).squeeze(1) + 1
            cu = torch.cat([torch.zeros(1, dtype=ends.dtype, device=ends.device), ends]).to(torch.int32)
        return pos_ids, cu

    def _loss_mask(self, input_ids, labels, loss_mask):
        mask = (labels != IGNORE_INDEX)
        if loss_mask is not None:
            mask = mask & (loss_mask.to(torch.bool))
        m = self.config.model
        if self.eod_mask_loss:
            # the masked positions are those whose *target* is the end-of-document or the padding token
            # (ironcore/language_model.py:118-125), not those whose input is
            for tok in (m.eod_token_id, m.pad_token_id):
                if tok is not None:
                    mask = mask & (labels != tok)
        return mask

    def hidden_states(self, input_ids, position_ids=None, cu_seqlens=None, attn_mask=None):
        """[B, S] ids -> normalised final hidden states, token-major (SP shard when enabled)."""
        b, s = input_ids.shape
        if position_ids is None and cu_seqlens is None:
            position_ids, cu_seqlens = self._document_layout(input_ids)
        pos_flat = position_ids.reshape(-1).to(torch.int32) if position_ids is not None else None
        x = self.embedding(input_ids, position_ids)
        x, aux = self.model(x, s, pos_flat, cu_seqlens, attn_mask)
        x = self.output_layernorm(x)
        return x, aux

    def logits_from_hidden(self, x: torch.Tensor) -> torch.Tensor:
        """token-major hidden [T(_local), d] -> vocab-sharded logits [T, V/t]."""
        if self.untied:
            return self.output_layer(x)
        if self.tp_size > 1:
            x = C.gather_from_sp(x, self.tp_group) if self.sequence_parallel else C.copy_to_tp(x, self.tp_group)
        return linear_t(x, self.embedding.word_embeddings.weight)

    def _head_chunk(self) -> int:
        """Vocabulary columns per step of the chunked LM head + cross entropy, or 0 for materialised logits:
        ``model.lm_head_chunk`` when set; without gradients (reference / old-policy log-probs, evaluation) the
        chunked form is chosen by itself for local vocabularies above 64 k entries, where the [tokens, vocab]
        matrix is the largest tensor of the pass and nothing needs it afterwards."""
        chunk = int(getattr(self.config.model, "lm_head_chunk", 0) or 0)
        if chunk > 0:
            return chunk
        v_local = self.padded_vocab_size // self.tp_size
        if not torch.is_grad_enabled() and v_local > 65536:
            return 8192
        return 0

    def per_token_loss(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Cross entropy of every token of the normalised final hidden states ``x`` (token-major, the
        sequence-parallel shard when enabled) against ``targets`` [T] (global ids, negative = ignored), fp32 [T].
        Chunked over the vocabulary when ``_head_chunk`` says so, through the logits otherwise."""
        chunk = self._head_chunk()
        if chunk <= 0:
            logits = self.logits_from_hidden(x)
            return vocab_parallel_cross_entropy(logits, targets, self.vocab_size, tp_group=self.tp_group)
        if self.tp_size > 1:
            x = C.gather_from_sp(x, self.tp_group) if self.sequence_parallel else C.copy_to_tp(x, self.tp_group)
        v_local = self.padded_vocab_size // self.tp_size
        start = mesh.get_tensor_model_parallel_rank() * v_local
        valid = max(0, min(v_local, self.vocab_size - start))
        if self.untied:
            weight, bias, tied = self.output_layer.weight, self.output_layer.bias, False
        else:
            weight, bias, tied = self.embedding.word_embeddings.weight, None, True
        return OF.chunked_head_cross_entropy(x, weight, targets, tied=tied, bias=bias, vocab_start=start,
                                             vocab_valid=valid, group=self.tp_group if self.tp_size > 1 else None,
                                             chunk=chunk)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None,
                loss_mask: Optional[torch.Tensor] = None, attn_mask: Optional[torch.Tensor] = None):
        dev = self.embedding.word_embeddings.weight.device
        if input_ids.device != dev:
            input_ids = input_ids.to(dev, non_blocking=True)
        if labels is not None and labels.device != dev:
            labels = labels.to(dev, non_blocking=True)
        b, s = input_ids.shape
        x, aux = self.hidden_states(input_ids, position_ids, cu_seqlens, attn_mask)
        if labels is None:
            return self.logits_from_hidden(x).view(b, s, -1)
        per_token = self.per_token_loss(x, labels.reshape(-1).clamp_min(-1))
        mask = self._loss_mask(input_ids, labels, loss_mask)
        loss = self.loss_fn(per_token.view(b, s), mask)
        if aux is not None:
            loss = loss + aux
        return loss

    def token_logprobs(self, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """log pi(labels[b, s] | input_ids[b, :s+1]) for every position, fp32 [B, S] (differentiable).
        The log-prob is the negative of the fused vocab-parallel cross entropy, so the
        ``[tokens, vocab]`` matrix is never expanded to fp32."""
        dev = self.embedding.word_embeddings.weight.device
        input_ids, labels = input_ids.to(dev), labels.to(dev)
        b, s = input_ids.shape
        x, _aux = self.hidden_states(input_ids)
        ce = self.per_token_loss(x, labels.reshape(-1).clamp_min(-1))
        return -ce.view(b, s)

    # ------------------------------------------------------------------ the reference's helper methods
    def get_masks_and_position_ids(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None):
        """``(attention_mask [B, 1, S, S] bool, position_ids [B, S], loss_mask [B, S] float)`` as the reference
        builds them for every batch (ironcore/language_model.py:102-161): causal mask, cut at document boundaries
        with ``reset_attention_mask``; positions restarting after an end-of-document token with
        ``reset_position_ids``; loss mask zero where the *label* is the end-of-document or padding token with
        ``eod_mask_loss``. ``forward`` does not need them (it hands document boundaries to the attention kernel);
        they serve callers that want the explicit tensors."""
        b, s = input_ids.shape
        dev = input_ids.device
        mask = torch.ones(s, s, dtype=torch.bool, device=dev).tril().expand(b, 1, s, s)
        pos, cu = self._document_layout(input_ids)
        if cu is not None:
            mask = mask & OF.document_mask(cu, b, s, dev)
        if pos is None:
            pos = torch.arange(s, device=dev).expand(b, s)
        loss_mask = torch.ones(b, s, dtype=torch.float, device=dev)
        m = self.config.model
        if self.eod_mask_loss and labels is not None:
            for tok in (m.eod_token_id, m.pad_token_id):
                if tok is not None:
                    loss_mask = loss_mask.masked_fill(labels == tok, 0.0)
        return mask, pos, loss_mask

    def compute_loss_from_logits(self, logits: torch.Tensor, labels: torch.Tensor, loss_mask: torch.Tensor,
                                 fp16_lm_cross_entropy: bool = False, padding_start_idx: Optional[int] = None):
        """Loss of (vocabulary-sharded) ``logits`` [B, S, V/t] against ``labels`` [B, S] through the
        vocab-parallel cross entropy and the model's loss function; labels of ``-100`` are left out.
        ``padding_start_idx`` defaults to the real vocabulary size. (ironcore/language_model.py:163-201)"""
        if not fp16_lm_cross_entropy and not OF.use_native(logits):
            logits = logits.float()      # (the native kernel reads 16-bit logits and computes in fp32 by itself)
        vocab = self.vocab_size if padding_start_idx is None else padding_start_idx
        per_token = vocab_parallel_cross_entropy(logits, labels.contiguous().clamp_min(-1), vocab,
                                                 tp_group=self.tp_group)
        mask = loss_mask.to(per_token.dtype) * (labels != IGNORE_INDEX).to(per_token.dtype)
        return self.loss_fn(per_token.view(labels.shape), mask)

    def post_lm_processing(self, lm_output: torch.Tensor, labels: Optional[torch.Tensor] = None,
                           loss_mask: Optional[torch.Tensor] = None, fp16_lm_cross_entropy: bool = False,
                           padding_start_idx: Optional[int] = None):
        """LM head on normalised hidden states ``[B, S, d]``: the (vocabulary-sharded) logits without labels, the
        loss with them. (ironcore/language_model.py:203-234)"""
        lead = lm_output.shape[:-1]
        logits = self.logits_from_hidden(lm_output.reshape(-1, lm_output.shape[-1]))
        logits = logits.view(*lead, -1) if logits.shape[0] == lead.numel() else logits
        if labels is None:
            return logits
        if loss_mask is None:
            loss_mask = torch.ones(labels.shape, dtype=torch.float, device=labels.device)
        return self.compute_loss_from_logits(logits.view(*labels.shape, -1), labels, loss_mask,
                                             fp16_lm_cross_entropy, padding_start_idx)

    def link_fused_norm_gather(self) -> int:
        """See ``TransformerModel.link_fused_norm_gather``; called once the fused tensor-parallel
        workspace has been attached to the parallel linears."""
        fn = getattr(self.model, "link_fused_norm_gather", None)
        return fn() if fn is not None else 0

    # ------------------------------------------------------------------ canonical (checkpoint) names
    def canonical_state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        """Local shard under the reference's parameter names: the fused ``linear_qkv`` is split
        into ``linear_q`` and ``linear_kv`` (K|V halves)."""
        out = OrderedDict()
        for name, t in self.state_dict().items():
            if ".linear_qkv." in name:
                layer = self.model.layers[int(name.split(".")[2])]
                qn = layer.heads_local * layer.head_dim
                q, kv = t.split([qn, t.shape[-1] - qn], dim=-1)
                out[name.replace("linear_qkv", "linear_q")] = q
                out[name.replace("linear_qkv", "linear_kv")] = kv
            else:
                out[name] = t
        return out

    def load_canonical_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True):
        fused = {}
        plain = {}
        for name, t in sd.items():
            name = name[7:] if name.startswith("module.") else name
            if ".linear_q." in name:
                fused.setdefault(name.replace("linear_q", "linear_qkv"), {})["q"] = t
            elif ".linear_kv." in name:
                fused.setdefault(name.replace("linear_kv", "linear_qkv"), {})["kv"] = t
            else:
                plain[name] = t
        for name, parts in fused.items():
            plain[name] = torch.cat([parts["q"], parts["kv"]], dim=-1)
        own = self.state_dict()
        for k in list(plain.keys()):
            if k in own and plain[k].shape != own[k].shape and plain[k].numel() == own[k].numel():
                plain[k] = plain[k].reshape(own[k].shape)
        return self.load_state_dict(plain, strict=strict)

    def canonical_shard_info(self) -> Dict[str, tuple]:
        """name -> (tp_shard_dim or None, parts) for every canonical tensor (used to merge /
        split universal checkpoints across TP sizes)."""
        info = {}
        params = dict(self.named_parameters())
        names = []
        for name in self.state_dict().keys():   # names only: parameter storage may be released (FSDP)
            if ".linear_qkv." in name:
                names += [name.replace("linear_qkv", "linear_q"), name.replace("linear_qkv", "linear_kv")]
            else:
                names.append(name)
        for name in names:
            if ".linear_q." in name:
                src = params[name.replace("linear_q", "linear_qkv")]
                info[name] = (getattr(src, "tp_shard_dim", None), 1)
            elif ".linear_kv." in name:
                src = params[name.replace("linear_kv", "linear_qkv")]
                info[name] = (getattr(src, "tp_shard_dim", None), 2)
            elif name in params:
                p = params[name]
                parts = getattr(p, "tp_parts", 1)
                info[name] = (getattr(p, "tp_shard_dim", None), parts if isinstance(parts, int) else 1)
            else:
                info[name] = (None, 1)
        return info
