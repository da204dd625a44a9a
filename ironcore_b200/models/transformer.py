"""The unified decoder stack.

One ``TransformerLayer`` class serves GPT-2 / Llama / Gemma / Qwen / Phi shapes through
configuration: pre- or post-norm residual topology, LayerNorm or RMSNorm, MHA / GQA / MQA,
rotary or learned positions, plain or gated MLP, optional parallel (Phi) block and a
mixture-of-experts feed-forward. Activations are token-major ``[T, d]`` (``T = batch *
seq``; a token shard under sequence parallelism), so norms, residuals and dropout run on
shards and the column / row parallel projections own the gather / reduce-scatter.

Internally q, k and v are one fused projection (``linear_qkv``: one gather, one GEMM);
checkpoints use the canonical ``linear_q`` / ``linear_kv`` tensors.
(Behavioural reference: ironcore/models/transformer.py:23-162.)
"""

from __future__ import annotations


import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..layers.attention import Attention
from ..layers.mlp import MLP
from ..layers.norm import get_norm
from ..layers.positional import RotaryPositionalEmbedding
from ..parallel import mesh
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, divide


class TransformerLayer(nn.Module):
    def __init__(self, config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        m = config.model
        tp = mesh.get_tensor_model_parallel_world_size()
        self.layer_idx = layer_idx
        self.d_model = m.d_model
        self.head_dim = m.head_dim
        self.num_heads = m.num_attention_heads
        self.num_kv_heads = m.num_attention_groups
        self.heads_local = divide(self.num_heads, tp)
        self.kv_heads_local = divide(self.num_kv_heads, tp)
        self.post_ln = m.post_ln
        self.parallel_block = bool(m.parallel_block)
        self.dropout_attn = m.dropout_attn
        q_out = self.num_heads * self.head_dim
        kv_out = self.num_kv_heads * self.head_dim
        self.input_layernorm = get_norm(config, dtype, device)
        self.linear_qkv = ColumnParallelLinear(m.d_model, q_out + 2 * kv_out, bias=bool(m.qkv_bias),
                                               concatenated_weights=[q_out, kv_out, kv_out], dtype=dtype, device=device)
        self.attn_output = RowParallelLinear(q_out, m.d_model, bias=not m.no_bias, input_is_parallel=True,
                                             dtype=dtype, device=device)
        rotary = None
        if m.positional_embedding.type.lower() == "rope":
            pe = m.positional_embedding
            rotary = RotaryPositionalEmbedding(self.head_dim, pe.base, pe.scaling_factor, pe.offset, pe.interleaved,
                                               float(pe.rotary_fraction or 1.0))
        self.rotary_pos_emb = rotary
        self.attention = Attention(self.heads_local, self.kv_heads_local, self.head_dim, dropout=m.dropout_attn,
                                   fused=config.trainer.use_flash_attn, causal=True, rotary=rotary)
        if not self.parallel_block:
            self.post_attn_layernorm = get_norm(config, dtype, device)
        moe = m.moe
        if moe.num_experts > 0 and (layer_idx % max(moe.layer_freq, 1) == 0):
            from .moe import MoEBlock

            self.mlp = MoEBlock(config, dtype=dtype, device=device)
            self.is_moe = True
        else:
            self.mlp = MLP(m.d_model, m.d_ffn, m.activation_type, bias=not m.no_bias, dropout=m.dropout_mlp,
                           dtype=dtype, device=device)
            self.is_moe = False

        # set by ``LanguageModel.link_fused_norm_gather``: fuse reduce-scatter + norm + gather across the
        # two norm boundaries this layer owns (attention output -> MLP, MLP output -> next layer)
        self.fuse_norm_gather = False
        self._next_layer = None

    def _attend(self, normed, seq_len, pos_ids, cu_seqlens, attn_mask, residual, pregathered=False):
        qkv = self.linear_qkv(normed, pregathered=True) if pregathered else self.linear_qkv(normed)
        ctx = self.attention(qkv, seq_len, pos_ids=pos_ids, cu_seqlens=cu_seqlens, attn_mask=attn_mask)
        if self.dropout_attn > 0 and self.training:
            out = F.dropout(self.attn_output(ctx), self.dropout_attn, True)
            return out if residual is None else out + residual
        return self.attn_output(ctx, residual=residual)

    def set_next_layer(self, layer):
        object.__setattr__(self, "_next_layer", layer)   # a plain reference, not a registered submodule

    def _forward_fused(self, x, seq_len, pos_ids, cu_seqlens, attn_mask, qkv):
        """Pre-norm dense layer with both norm boundaries fused into the GEMM kernels around them:
        attention output -> (reduce-scatter + residual + post-attention norm + gather) -> MLP up projection, and
        MLP down projection -> (reduce-scatter + residual + next layer's input norm + gather) -> next layer's
        qkv projection, which this layer hands over."""
        if qkv is None:
            qkv = self.linear_qkv(self.input_layernorm(x, out=self.linear_qkv.gather_target(x)))
        ctx = self.attention(qkv, seq_len, pos_ids=pos_ids, cu_seqlens=cu_seqlens, attn_mask=attn_mask)
        up = self.mlp.up_proj
        if self.attn_output.can_fuse_norm(ctx, self.post_attn_layernorm, up):
            h, up_out = self.attn_output.forward_norm_linear(ctx, x, self.post_attn_layernorm, up)
        else:
            h = self.attn_output(ctx, residual=x)
            up_out = up(self.post_attn_layernorm(h, out=up.gather_target(h)))
        nxt = self._next_layer
        if nxt is not None and nxt.fuse_norm_gather:
            out, next_qkv = self.mlp(None, residual=h, up_out=up_out, next_norm=nxt.input_layernorm,
                                     next_consumer=nxt.linear_qkv)
        else:
            out, next_qkv = self.mlp(None, residual=h, up_out=up_out), None
        return out, None, next_qkv

    def forward(self, x: torch.Tensor, seq_len: int, pos_ids=None, cu_seqlens=None, attn_mask=None, prenormed=None):
        """x: [T_local, d]. Returns (x, aux_loss or None, qkv_for_next_layer or None). ``prenormed``:
        this layer's qkv projection of its input norm of ``x``, computed by the previous layer inside its
        fused output boundary."""
        if self.fuse_norm_gather and self.dropout_attn == 0:
            return self._forward_fused(x, seq_len, pos_ids, cu_seqlens, attn_mask, prenormed)
        aux = None
        # (not under post-norm, where the normalised tensor lives on as the residual)
        n1 = self.input_layernorm(x, out=None if self.post_ln else self.linear_qkv.gather_target(x))
        if self.parallel_block:
            a = self._attend(n1, seq_len, pos_ids, cu_seqlens, attn_mask, residual=x)
            out = self.mlp(n1, residual=a)
            if self.is_moe:
                out, aux = out
            return out, aux, None
        res1 = n1 if self.post_ln else x
        x = self._attend(n1, seq_len, pos_ids, cu_seqlens, attn_mask, residual=res1)
        up = getattr(self.mlp, "up_proj", None)
        n2 = self.post_attn_layernorm(x, out=up.gather_target(x) if (up is not None and not self.post_ln) else None)
        res2 = n2 if self.post_ln else x
        out = self.mlp(n2, residual=res2)
        if self.is_moe:
            out, aux = out
        return out, aux, None


class TransformerModel(nn.Module):
    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([TransformerLayer(config, i, dtype, device) for i in range(config.model.num_layers)])
        self.recompute = config.operation.activation_recompute
        self.use_reentrant = config.operation.recompute_strategy == "optimized"

    def link_fused_norm_gather(self) -> int:
        """Mark the layers whose norm boundaries can run inside the preceding row-parallel GEMM kernel
        (pre-norm dense layers with RMSNorm, no dropout, fused workspace attached, no activation
        recompute) and chain them. Returns the number of marked layers."""
        n = 0
        prev = None
        for layer in self.layers:
            ok = (not self.recompute and not layer.is_moe and not layer.parallel_block and not layer.post_ln
                  and layer.dropout_attn == 0 and getattr(layer.mlp, "dropout", 0) == 0
                  and getattr(layer.input_layernorm, "rms", False) and layer.input_layernorm.layernorm.bias is None
                  and getattr(layer.linear_qkv, "gather_slot", None) is not None
                  and getattr(layer.mlp.up_proj, "gather_slot", None) is not None
                  and getattr(layer.attn_output, "fused", None) is not None)
            layer.fuse_norm_gather = bool(ok)
            layer.set_next_layer(None)
            if prev is not None and prev.fuse_norm_gather:
                prev.set_next_layer(layer)
            prev = layer
            n += int(ok)
        return n

    def forward(self, x, seq_len: int, pos_ids=None, cu_seqlens=None, attn_mask=None):
        aux_total = None
        prenormed = None
        for layer in self.layers:
            if self.recompute and self.training:
                x, aux, prenormed = checkpoint(layer, x, seq_len, pos_ids, cu_seqlens, attn_mask,
                                               use_reentrant=self.use_reentrant)
            else:
                x, aux, prenormed = layer(x, seq_len, pos_ids, cu_seqlens, attn_mask, prenormed)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        return x, aux_total
