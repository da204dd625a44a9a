"""Rollout engine: prefill + decode over the block KV cache with the model's own weights.

Prefill runs the flash attention kernel on the packed projections and scatters the rotated K / V
rows into cache pages; every decode step appends one token per sequence and attends over its pages
with the paged decode kernel. Tensor parallelism uses the plain (non sequence-parallel) layout —
one all-reduce after each row-parallel projection — because a decode step has only ``num_seqs``
tokens. The decode step runs on static buffers, so it can be captured once in a CUDA graph and
replayed (launch-bound regime: dozens of small kernels per layer).
(The reference only has a cache-less sampler that re-runs the whole prefix for every token:
examples/generate_text.py:12-46.)
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import kernels
from ..parallel import mesh
from . import ops as RO
from .kv_cache import BlockKVCache
from .sampling import sample_tokens


def _all_reduce(x, group):
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, group=group)
    return x


class RolloutEngine:
    def __init__(self, model, config, max_seqs: int, max_seq_len: int, block_size: Optional[int] = None,
                 use_cuda_graph: Optional[bool] = None):
        self.model = model
        self.config = config
        m = config.model
        self.tp_group = mesh.get_tensor_model_parallel_group()
        self.tp = mesh.get_tensor_model_parallel_world_size()
        self.tp_rank = mesh.get_tensor_model_parallel_rank()
        self.hq = m.num_attention_heads // self.tp
        self.hkv = (m.num_attention_groups or m.num_attention_heads) // self.tp
        self.hd = m.head_dim
        self.d = m.d_model
        self.layers = list(model.model.layers)
        dev = next(model.parameters()).device
        self.device = dev
        self.dtype = next(model.parameters()).dtype
        bs = block_size or config.rl.kv_block_size
        blocks = max_seqs * ((max_seq_len + bs - 1) // bs)
        self.cache = BlockKVCache(len(self.layers), self.hkv, self.hd, blocks, bs, max_seqs, max_seq_len, self.dtype, dev)
        self.max_seqs = max_seqs
        self.use_graph = (dev.type == "cuda") if use_cuda_graph is None else (use_cuda_graph and dev.type == "cuda")
        self._graph = None
        self._static_tokens = None
        self._static_logits = None
        self._graph_seqs = 0

    # ------------------------------------------------------------------ building blocks
    def _embed(self, ids_2d: torch.Tensor, pos_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        emb = self.model.embedding
        w = emb.word_embeddings
        pt = emb.position_embedding.weight if emb.position_embedding is not None else None
        if self.tp > 1:
            x = OF.embedding(ids_2d, w.weight, vocab_start=w.vocab_start, pos_table=pt if self.tp_rank == 0 else None,
                             pos_ids=pos_ids)
            x = _all_reduce(x.reshape(-1, self.d).contiguous(), self.tp_group)
        else:
            x = OF.embedding(ids_2d, w.weight, pos_table=pt, pos_ids=pos_ids).reshape(-1, self.d)
        if emb.scale is not None:
            x = x * emb.scale
        return x

    def _row_parallel(self, lin, x, residual):
        if self.tp == 1:
            return OF.linear(x, lin.weight, lin.bias, residual)
        y = OF.linear(x, lin.weight, None)
        y = _all_reduce(y, self.tp_group)
        if lin.bias is not None:
            y = y + lin.bias
        return y + residual if residual is not None else y

    def _mlp(self, layer, x, residual):
        mlp = layer.mlp
        if getattr(layer, "is_moe", False):
            out, _aux = mlp(x, residual=residual)
            return out
        h = mlp.activation(OF.linear(x, mlp.up_proj.weight, mlp.up_proj.bias))
        return self._row_parallel(mlp.down_proj, h, residual)

    def _layer(self, li: int, layer, x, attend):
        n1 = layer.input_layernorm(x)
        qkv = OF.linear(n1, layer.linear_qkv.weight, layer.linear_qkv.bias)
        ctx = attend(li, layer, qkv)
        if layer.parallel_block:
            a = self._row_parallel(layer.attn_output, ctx, x)
            return self._mlp(layer, n1, a)
        res1 = n1 if layer.post_ln else x
        x = self._row_parallel(layer.attn_output, ctx, res1)
        n2 = layer.post_attn_layernorm(x)
        res2 = n2 if layer.post_ln else x
        return self._mlp(layer, n2, res2)

    def _rope_inplace(self, layer, qkv, tokens: int, seq_len: int, pos_ids):
        rot = layer.rotary_pos_emb
        if rot is None:
            return qkv
        if OF.use_native(qkv) and rot.rot_dim % 2 == 0:
            kernels.rope(qkv, qkv, nheads=self.hq + self.hkv, head_dim=self.hd, tokens=tokens, seq_len=seq_len,
                         base=rot.base, scale=rot.scaling_factor, offset=rot.offset, interleaved=rot.interleaved,
                         pos_ids=pos_ids, row_stride=qkv.stride(0), out_stride=qkv.stride(0), rot_dim=rot.rot_dim)
            return qkv
        return OF.rope_reference_packed(qkv, self.hq, self.hkv, self.hd, seq_len, rot.base, rot.scaling_factor,
                                        rot.offset, rot.interleaved, rot.rot_dim, pos_ids)

    def _logits(self, x):
        x = self.model.output_layernorm(x)
        if self.model.untied:
            ol = self.model.output_layer
            return OF.linear(x, ol.weight, ol.bias)
        from ..models.language_model import linear_t

        return linear_t(x, self.model.embedding.word_embeddings.weight)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        """prompts [S, P] -> logits of the last prompt position [S, V_local]; fills the cache."""
        s, p = prompts.shape
        cache = self.cache
        cache.reset()
        cache.reserve_all(s, p)
        prompts = prompts.to(self.device)
        seq_ids = torch.arange(s, device=self.device).repeat_interleave(p)
        pos = torch.arange(p, device=self.device).repeat(s)
        slots = cache.slots_for(seq_ids, pos)
        q_cols = self.hq * self.hd
        kv_cols = self.hkv * self.hd

        def attend(li, layer, qkv):
            qkv = self._rope_inplace(layer, qkv, s * p, p, None)
            RO.kv_append(qkv[:, q_cols:q_cols + kv_cols], qkv[:, q_cols + kv_cols:], cache.k[li], cache.v[li], slots)
            return OF.rope_attention(qkv, num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.hd, seq_len=p,
                                     rope=None, causal=True, fused=self.config.trainer.use_flash_attn)

        x = self._embed(prompts)
        for li, layer in enumerate(self.layers):
            x = self._layer(li, layer, x, attend)
        cache.seq_lens[:s] = p
        last = x.view(s, p, self.d)[:, -1].contiguous()
        return self._logits(last)

    # ------------------------------------------------------------------ decode
    def _decode_body(self, tokens: torch.Tensor, s: int) -> torch.Tensor:
        cache = self.cache
        lens = cache.seq_lens[:s]
        pos = lens.to(torch.int32)
        seq_ids = torch.arange(s, device=self.device)
        slots = cache.slots_for(seq_ids, pos.long())
        q_cols = self.hq * self.hd
        kv_cols = self.hkv * self.hd
        new_lens = (lens + 1).to(torch.int32)

        def attend(li, layer, qkv):
            qkv = self._rope_inplace(layer, qkv, s, 1, pos)
            RO.kv_append(qkv[:, q_cols:q_cols + kv_cols], qkv[:, q_cols + kv_cols:], cache.k[li], cache.v[li], slots)
            return RO.paged_decode(qkv[:, :q_cols], cache.k[li], cache.v[li], cache.block_table, new_lens, self.hq,
                                   self.hkv, self.hd)

        pos_for_emb = pos.view(s, 1) if self.model.embedding.position_embedding is not None else None
        x = self._embed(tokens.view(s, 1), pos_for_emb)
        for li, layer in enumerate(self.layers):
            x = self._layer(li, layer, x, attend)
        logits = self._logits(x)
        cache.seq_lens[:s] = new_lens
        return logits

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, cur_len: int) -> torch.Tensor:
        """Append ``tokens`` [S] (position ``cur_len`` of every sequence) and return next-token logits."""
        s = tokens.shape[0]
        self.cache.reserve_all(s, cur_len + 1)
        if not self.use_graph:
            return self._decode_body(tokens.to(self.device), s)
        if self._graph is None or self._graph_seqs != s:
            self._static_tokens = torch.zeros(s, dtype=torch.int64, device=self.device)
            self._static_tokens.copy_(tokens)
            # warm up on a side stream (allocator, lazy kernel attributes), restoring the lengths afterwards
            saved = self.cache.seq_lens.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._decode_body(self._static_tokens, s)
            torch.cuda.current_stream().wait_stream(side)
            self.cache.seq_lens.copy_(saved)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._static_logits = self._decode_body(self._static_tokens, s)
            self.cache.seq_lens.copy_(saved)
            self._graph_seqs = s
        self._static_tokens.copy_(tokens)
        self._graph.replay()
        return self._static_logits

    def release_graph(self):
        """Drop the captured decode step (and its static buffers); the next ``decode_step`` captures again."""
        if self._graph is not None:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._graph = None
            self._static_logits = None
            self._static_tokens = None
            self._graph_seqs = 0
            import gc

            gc.collect()

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns (tokens [S, P + N] including the prompt, log-probs of the N sampled tokens [S, N])."""
        was_training = self.model.training
        self.model.eval()
        s, p = prompts.shape
        vocab_local = self.model.padded_vocab_size // self.tp
        start = self.tp_rank * vocab_local
        valid = max(0, min(vocab_local, self.model.vocab_size - start))
        out = torch.empty((s, p + max_new_tokens), dtype=torch.int64, device=self.device)
        out[:, :p] = prompts.to(self.device)
        logps = torch.empty((s, max_new_tokens), dtype=torch.float32, device=self.device)
        logits = self.prefill(prompts)
        for i in range(max_new_tokens):
            tok, lp = sample_tokens(logits, temperature, top_k, top_p, generator, vocab_start=start, vocab_valid=valid,
                                    group=self.tp_group if self.tp > 1 else None)
            out[:, p + i] = tok
            logps[:, i] = lp
            if i + 1 < max_new_tokens:
                logits = self.decode_step(tok, p + i)
        if was_training:
            self.model.train()
        return out, logps
