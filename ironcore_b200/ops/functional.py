"""Differentiable ops. On CUDA every op launches the native sm_100a kernels; on CPU
(and for dtypes the kernels do not cover, i.e. fp32) the same math runs as plain
PyTorch — that path is the numerical oracle of the GPU tests and the CPU execution
path of the framework. There is no silent fallback on a GPU: a CUDA tensor in a
16-bit dtype always takes the native path and raises if the library is missing.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import kernels, reference
from .kernels import ACT_KINDS, GLU_KINDS

_NATIVE_DTYPES = (torch.bfloat16, torch.float16)


def use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in _NATIVE_DTYPES


_FALLBACKS_SEEN = set()


def note_fallback(op: str, reason: str, t: Optional[torch.Tensor] = None) -> None:
    """A 16-bit CUDA tensor is about to run ``op`` through PyTorch operators instead of the native kernel because
    its shape is outside the kernel's range: say so, once per (op, reason), so that the slow path never runs
    unnoticed. Tensors for which the native path was never an option (CPU, fp32) are not reported."""
    if t is not None and not use_native(t):
        return
    key = (op, reason)
    if key in _FALLBACKS_SEEN:
        return
    _FALLBACKS_SEEN.add(key)
    import warnings

    warnings.warn(f"{op}: {reason}; this call runs on PyTorch operators, not on the native sm_100a kernel",
                  RuntimeWarning, stacklevel=3)


# --------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    """y = x @ W (+ b) (+ residual) with W stored [in, out]."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, weight.shape[1])
        y = kernels.mm_nn(x2, weight, bias=bias, residual=res2)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.in_shape = shape
        return y.view(*shape[:-1], weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, weight.shape[1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx = kernels.mm_nt(dy2, weight).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                # accumulate straight into the flat gradient buffer (C += x^T dy in the GEMM epilogue)
                kernels.mm_tn(x2, dy2, out=main_grad, residual=main_grad, out_dtype=main_grad.dtype)
                weight.grad_ready = True
                dw = None
            else:
                dw = kernels.mm_tn(x2, dy2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(dy.dtype)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if use_native(x):
        return _Linear.apply(x, weight, bias, residual)
    y = x @ weight
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    return y


# --------------------------------------------------------------------------- norm
class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, eps, rms, w_offset, out=None):
        y, h, mean, rstd = kernels.norm_fwd(x, weight, bias, eps, rms, residual=residual, w_offset=w_offset, out=out)
        ctx.save_for_backward(h, weight, mean if mean is not None else rstd, rstd)
        ctx.rms = rms
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.w_offset = w_offset
        if residual is not None:
            return y, h
        return y, x

    @staticmethod
    def backward(ctx, dy, dh):
        h, weight, mean, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        dres_in = dh.contiguous() if (ctx.has_res and dh is not None) else None
        dx, dw, db = kernels.norm_bwd(dy, h, weight, None if ctx.rms else mean, rstd, ctx.rms, ctx.has_bias,
                                      dres_in=dres_in, w_offset=ctx.w_offset)
        dwt = dw.to(weight.dtype)
        dbt = db.to(weight.dtype) if db is not None else None
        if ctx.has_res:
            return dx, dwt, dbt, dx, None, None, None, None
        if dh is not None:
            dx = dx + dh
        return dx, dwt, dbt, None, None, None, None, None


def norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, rms: bool,
         residual: Optional[torch.Tensor] = None, w_offset: float = 0.0,
         out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(normalised, h)`` with ``h = x + residual`` (or ``x`` when no residual):
    the (fused) residual add and the norm that follows it. ``out`` (native path, 2-D input only): where the
    normalised rows are written, e.g. this rank's rows of the gather buffer of the next linear."""
    if use_native(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        xc = x if x.is_contiguous() else x.contiguous()
        rc = residual
        if rc is not None and not rc.is_contiguous():
            rc = rc.contiguous()
        if out is not None and (xc.dim() != 2 or out.shape != xc.shape or out.dtype != xc.dtype):
            out = None
        return _Norm.apply(xc, weight, bias, rc, eps, rms, w_offset, out)
    note_fallback("norm", f"row length {x.shape[-1]} is not a multiple of 8 up to 8192", x)
    h = x if residual is None else x + residual
    if rms:
        y = reference.rms_norm_reference(h, weight, eps, w_offset)
    else:
        y = reference.layer_norm_reference(h, weight, bias, eps)
    return y, h


# --------------------------------------------------------------------------- activations
class _Glu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name, row_limit=None):
        ctx.save_for_backward(x, row_limit if row_limit is not None else x)
        ctx.name = name
        ctx.limited = row_limit is not None
        return kernels.glu_fwd(x, name, row_limit)

    @staticmethod
    def backward(ctx, dy):
        x, limit = ctx.saved_tensors
        return kernels.glu_bwd(dy.contiguous(), x, ctx.name, limit if ctx.limited else None), None, None


class _Act(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):
        ctx.save_for_backward(x)
        ctx.name = name
        return kernels.act_fwd(x, name)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return kernels.act_bwd(dy, x, ctx.name).view(x.shape), None


def is_gated(name: str) -> bool:
    return name in GLU_KINDS


def _mask_rows(x: torch.Tensor, row_limit: torch.Tensor) -> torch.Tensor:
    row = torch.arange(x.shape[0], device=x.device)
    return torch.where((row < row_limit.to(torch.long))[:, None], x, torch.zeros((), dtype=x.dtype, device=x.device))


def activation(x: torch.Tensor, name: str, row_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Plain (relu/gelu/gelu_tanh/silu) or gated (swiglu/geglu/reglu/glu on [f|g] halves) activation.

    ``row_limit`` (int32 device tensor with one element) declares the rows of a 2-D ``x`` from that index on as
    holding nothing: they come out as zeros and receive a zero gradient. The gated kernels neither read nor
    compute them; the other paths mask."""
    if name in GLU_KINDS:
        if use_native(x) and (x.shape[-1] // 2) % 8 == 0:
            return _Glu.apply(x.contiguous(), name, row_limit)
        note_fallback("gated activation", f"half width {x.shape[-1] // 2} is not a multiple of 8", x)
        if row_limit is not None:
            x = _mask_rows(x, row_limit)
        return reference.glu_reference(x, name)
    if row_limit is not None:
        x = _mask_rows(x, row_limit)
    if name not in ACT_KINDS:
        raise ValueError(f"unknown activation type {name}")
    if use_native(x) and x.numel() % 8 == 0:
        return _Act.apply(x.contiguous(), name)
    note_fallback("activation", f"element count {x.numel()} is not a multiple of 8", x)
    return reference.act_reference(x, name)


# --------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, pos_table, pos_ids, vocab_start, seq_len):
        out = kernels.embedding_fwd(ids, weight, vocab_start=vocab_start, pos_table=pos_table, pos_ids=pos_ids,
                                    seq_len=seq_len)
        ctx.save_for_backward(ids, pos_ids if pos_ids is not None else ids)
        ctx.has_pos_ids = pos_ids is not None
        ctx.vocab_start = vocab_start
        ctx.seq_len = seq_len
        ctx.rows = weight.shape[0]
        ctx.w_dtype = weight.dtype
        ctx.pos_rows = pos_table.shape[0] if pos_table is not None else 0
        ctx.weight_ref = weight
        return out

    @staticmethod
    def backward(ctx, dy):
        ids, pos_saved = ctx.saved_tensors
        main_grad = getattr(ctx.weight_ref, "main_grad", None)
        if main_grad is not None and main_grad.dtype == torch.float32:
            # scatter-add straight into the flat fp32 gradient buffer: no [V, d] temporary, no conversion
            kernels.embedding_bwd(ids, dy, ctx.rows, row_start=ctx.vocab_start, out=main_grad)
            ctx.weight_ref.grad_ready = True
            dw = None
        else:
            dw = kernels.embedding_bwd(ids, dy, ctx.rows, row_start=ctx.vocab_start).to(ctx.w_dtype)
        dpos = None
        if ctx.pos_rows:
            if ctx.has_pos_ids:
                pos = pos_saved.reshape(-1).long()
            else:
                pos = (torch.arange(ids.numel(), device=ids.device) % ctx.seq_len)
            dpos = kernels.embedding_bwd(pos, dy, ctx.pos_rows).to(ctx.w_dtype)
        return None, dw, dpos, None, None, None


def embedding(ids: torch.Tensor, weight: torch.Tensor, *, vocab_start: int = 0,
              pos_table: Optional[torch.Tensor] = None, pos_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token (+ learned position) embedding for ids [B, S]; ids outside this shard's rows give zeros."""
    seq_len = ids.shape[-1]
    if use_native(weight) and weight.shape[1] % 8 == 0:
        pid = pos_ids.reshape(-1).to(torch.int32) if pos_ids is not None else None
        return _Embedding.apply(ids, weight, pos_table, pid, vocab_start, seq_len)
    local = ids - vocab_start
    ok = (local >= 0) & (local < weight.shape[0])
    out = F.embedding(local.clamp(0, weight.shape[0] - 1), weight)
    out = out * ok.unsqueeze(-1).to(out.dtype)
    if pos_table is not None:
        if pos_ids is None:
            pos_ids = torch.arange(seq_len, device=ids.device).expand_as(ids)
        out = out + F.embedding(pos_ids.long(), pos_table)
    return out


# --------------------------------------------------------------------------- cross entropy
class _CrossEntropy(torch.autograd.Function):
    """Per-token loss over a (vocab-sharded) logits matrix. The backward pass overwrites the
    logits buffer with the gradient (the buffer is owned by this op's caller chain)."""

    @staticmethod
    def forward(ctx, logits, targets, vocab_start, vocab_valid, group):
        rmax, rsum, rtgt = kernels.ce_stats(logits, targets, vocab_start=vocab_start, vocab_valid=vocab_valid)
        if group is not None and torch.distributed.get_world_size(group) > 1:
            import torch.distributed as dist

            gmax = rmax.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack([rsum * torch.exp(rmax - gmax), rtgt])
            dist.all_reduce(packed, group=group)
            rsum, rtgt, rmax = packed[0], packed[1], gmax
        lse = rmax + torch.log(rsum)
        loss = lse - rtgt
        ignore = targets < 0
        loss = loss.masked_fill(ignore, 0.0)
        ctx.save_for_backward(logits, targets, lse)
        ctx.vocab_start = vocab_start
        ctx.vocab_valid = vocab_valid
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, targets, lse = ctx.saved_tensors
        gs = dloss.float().masked_fill(targets < 0, 0.0).contiguous()
        g = kernels.ce_grad_(logits, targets, lse, gs, vocab_start=ctx.vocab_start, vocab_valid=ctx.vocab_valid)
        return g, None, None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, *, vocab_start: int = 0,
                  vocab_valid: Optional[int] = None, group=None) -> torch.Tensor:
    """Per-token cross entropy. ``logits`` [T, V_local]; targets [T] global ids (negative = ignored).
    With ``group`` the vocab is sharded over the group (vocab_start = first id of this shard);
    columns >= vocab_valid of the local shard are padding. Returns fp32 [T]."""
    t, v = logits.shape
    vv = v if vocab_valid is None else vocab_valid
    if use_native(logits) and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        return _CrossEntropy.apply(logits, targets.contiguous(), vocab_start, vv, group)
    lf = logits.float()
    if vv < v:
        pad = torch.arange(v, device=logits.device) >= vv
        lf = lf.masked_fill(pad, float("-inf"))
    local_t = targets - vocab_start
    mine = (local_t >= 0) & (local_t < vv)
    rmax = lf.max(dim=-1).values
    if group is not None and torch.distributed.get_world_size(group) > 1:
        import torch.distributed as dist

        gmax = rmax.detach().clone()
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        from ..parallel.collectives import all_reduce_sum

        sumexp = all_reduce_sum(torch.exp(lf - gmax[:, None]).sum(-1), group)
        tgt = lf.gather(1, local_t.clamp(0, max(vv - 1, 0))[:, None]).squeeze(1).masked_fill(~mine, 0.0)
        tgt = all_reduce_sum(tgt, group)
        loss = torch.log(sumexp) + gmax - tgt
    else:
        gmax = rmax.detach()
        sumexp = torch.exp(lf - gmax[:, None]).sum(-1)
        tgt = lf.gather(1, local_t.clamp(0, max(vv - 1, 0))[:, None]).squeeze(1).masked_fill(~mine, 0.0)
        loss = torch.log(sumexp) + gmax - tgt
    return loss.masked_fill(targets < 0, 0.0)


# --------------------------------------------------------------------------- LM head + cross entropy, chunked
def _head_chunk_logits(x, weight, bias, tied, c0, c1, buf, native_path):
    """logits of vocabulary columns [c0, c1): x [T, d] times the head's slice, into ``buf[:, :c1 - c0]``."""
    n = c1 - c0
    b = bias[c0:c1] if bias is not None else None
    if native_path:
        out = buf[:, :n]
        if tied:     # weight [V, d]: rows are vocabulary entries
            kernels.gemm(x, weight[c0:c1], a_major=0, b_major=0, m=x.shape[0], n=n, k=x.shape[1], out=out, bias=b)
        else:        # weight [d, V]
            kernels.gemm(x, weight[:, c0:c1], a_major=0, b_major=1, m=x.shape[0], n=n, k=x.shape[1], out=out, bias=b)
        return out
    w = weight[c0:c1].t() if tied else weight[:, c0:c1]
    y = x @ w
    return y + b if b is not None else y


def _head_chunk_stats(logits, targets, start, valid, native_path):
    """(row max, sum of exp(logit - max), target logit or 0) over the chunk's first ``valid`` columns; ``start`` is
    the global id of its first column."""
    if native_path:
        return kernels.ce_stats(logits, targets, vocab_start=start, vocab_valid=valid)
    lf = logits.float()[:, :valid]
    cm = lf.max(dim=-1).values
    cs = torch.exp(lf - cm[:, None]).sum(-1)
    local = targets - start
    mine = (local >= 0) & (local < valid)
    ct = lf.gather(1, local.clamp(0, valid - 1)[:, None]).squeeze(1) * mine.to(lf.dtype)
    return cm, cs, ct


def _head_chunk_grad_(logits, targets, lse, gs, start, valid, native_path):
    """d loss / d logits of the chunk: gs * (softmax - one_hot(target)); zero for padding columns."""
    if native_path:
        return kernels.ce_grad_(logits, targets, lse, gs, vocab_start=start, vocab_valid=valid)
    lf = logits.float()
    g = torch.exp(lf - lse[:, None])
    g[:, valid:] = 0.0
    local = targets - start
    mine = (local >= 0) & (local < valid)
    rows = torch.nonzero(mine).squeeze(1)
    g[rows, local[rows]] -= 1.0
    return (g * gs[:, None]).to(logits.dtype)


class _ChunkedHeadCE(torch.autograd.Function):
    """LM head and cross entropy over chunks of the (local) vocabulary. Logits exist only as one [T, chunk] block at a
    time: the forward pass runs GEMM + row statistics per chunk and merges the statistics the way vocabulary shards
    of a tensor-parallel group are merged; the backward pass recomputes a chunk's logits, turns them into their
    gradient in place and feeds the dX and dW GEMMs from it. One more GEMM than the materialised form, no
    [T, V] tensor."""

    @staticmethod
    def forward(ctx, x, weight, bias, targets, tied, vocab_start, vocab_valid, group, chunk):
        native_path = use_native(x)
        t = x.shape[0]
        v_local = weight.shape[0] if tied else weight.shape[1]
        x = x.contiguous()
        targets = targets.contiguous()
        rmax = torch.full((t,), float("-inf"), dtype=torch.float32, device=x.device)
        rsum = torch.zeros(t, dtype=torch.float32, device=x.device)
        rtgt = torch.zeros(t, dtype=torch.float32, device=x.device)
        buf = torch.empty((t, chunk), dtype=x.dtype, device=x.device) if native_path else None
        for c0 in range(0, v_local, chunk):
            c1 = min(c0 + chunk, v_local)
            valid = max(0, min(c1 - c0, vocab_valid - c0))
            if valid == 0:
                break
            logits = _head_chunk_logits(x, weight, bias, tied, c0, c1, buf, native_path)
            cm, cs, ct = _head_chunk_stats(logits, targets, vocab_start + c0, valid, native_path)
            new = torch.maximum(rmax, cm)
            rsum = rsum * torch.exp(rmax - new) + cs * torch.exp(cm - new)
            rtgt = rtgt + ct
            rmax = new
        if group is not None and torch.distributed.get_world_size(group) > 1:
            import torch.distributed as dist

            gmax = rmax.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack([rsum * torch.exp(rmax - gmax), rtgt])
            dist.all_reduce(packed, group=group)
            rsum, rtgt, rmax = packed[0], packed[1], gmax
        lse = rmax + torch.log(rsum)
        loss = (lse - rtgt).masked_fill(targets < 0, 0.0)
        ctx.save_for_backward(x, weight, bias if bias is not None else lse, targets, lse)
        ctx.meta = (tied, vocab_start, vocab_valid, chunk, bias is not None, native_path)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x, weight, bias, targets, lse = ctx.saved_tensors
        tied, vocab_start, vocab_valid, chunk, has_bias, native_path = ctx.meta
        bias = bias if has_bias else None
        t, d = x.shape
        v_local = weight.shape[0] if tied else weight.shape[1]
        gs = dloss.float().masked_fill(targets < 0, 0.0).contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        main_grad = getattr(weight, "main_grad", None) if need_dw else None
        dx_acc = torch.zeros((t, d), dtype=torch.float32, device=x.device) if need_dx else None
        dw = torch.zeros_like(weight) if (need_dw and main_grad is None) else None
        db = torch.zeros_like(bias) if (has_bias and ctx.needs_input_grad[2]) else None
        buf = torch.empty((t, chunk), dtype=x.dtype, device=x.device) if native_path else None
        for c0 in range(0, v_local, chunk):
            c1 = min(c0 + chunk, v_local)
            n = c1 - c0
            valid = max(0, min(n, vocab_valid - c0))
            if valid == 0:
                break
            logits = _head_chunk_logits(x, weight, bias, tied, c0, c1, buf, native_path)
            dl = _head_chunk_grad_(logits, targets, lse, gs, vocab_start + c0, valid, native_path)
            w_c = weight[c0:c1] if tied else weight[:, c0:c1]
            if need_dx:
                if native_path:     # dx += dl @ W_c (tied: [n, d]) or dl @ W_c^T (untied: [d, n])
                    kernels.gemm(dl, w_c, a_major=0, b_major=1 if tied else 0, m=t, n=d, k=n, out=dx_acc,
                                 residual=dx_acc, out_dtype=torch.float32)
                else:
                    dx_acc += (dl.float() @ (w_c.float() if tied else w_c.float().t()))
            if need_dw:
                target = main_grad if main_grad is not None else dw
                tgt_c = target[c0:c1] if tied else target[:, c0:c1]
                if native_path:     # tied: dW_c [n, d] = dl^T x; untied: dW_c [d, n] = x^T dl
                    a, b_ = (dl, x) if tied else (x, dl)
                    kernels.gemm(a, b_, a_major=1, b_major=1, m=tgt_c.shape[0], n=tgt_c.shape[1], k=t, out=tgt_c,
                                 residual=tgt_c if main_grad is not None else None, out_dtype=tgt_c.dtype)
                else:
                    upd = (dl.float().t() @ x.float()) if tied else (x.float().t() @ dl.float())
                    tgt_c += upd.to(tgt_c.dtype)
            if db is not None:
                db[c0:c1] = dl.sum(0, dtype=torch.float32).to(db.dtype)
        if main_grad is not None:
            weight.grad_ready = True
        dx = dx_acc.to(x.dtype) if need_dx else None
        return dx, dw, db, None, None, None, None, None, None


def chunked_head_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, *, tied: bool,
                               bias: Optional[torch.Tensor] = None, vocab_start: int = 0,
                               vocab_valid: Optional[int] = None, group=None, chunk: int = 8192) -> torch.Tensor:
    """Per-token cross entropy of ``x`` [T, d] under the LM head ``weight`` ([V_local, d] when ``tied``: the
    embedding table; [d, V_local] otherwise) without the [T, V_local] logits: see ``_ChunkedHeadCE``. ``targets``
    [T] are global ids (negative = ignored); ``vocab_start`` is the first id of this rank's shard, columns from
    ``vocab_valid`` on are padding; ``chunk`` (a multiple of 128) columns are live at a time. Returns fp32 [T]."""
    v_local = weight.shape[0] if tied else weight.shape[1]
    if chunk % 128 or chunk <= 0:
        raise ValueError("chunk must be a positive multiple of 128")
    vv = v_local if vocab_valid is None else vocab_valid
    return _ChunkedHeadCE.apply(x, weight, bias, targets, bool(tied), int(vocab_start), int(vv), group, int(chunk))


# --------------------------------------------------------------------------- rope + attention
def _positions(tokens: int, seq_len: int, device, pos_ids=None):
    if pos_ids is not None:
        return pos_ids.reshape(-1)
    return torch.arange(tokens, device=device) % seq_len


def rope_reference_packed(qkv, hq, hkv, hd, seq_len, base, scale, offset, interleaved, rot_dim, pos_ids=None,
                          inverse=False):
    """Rotate the q and k heads of packed qkv [T, (hq+2hkv)*hd] (out of place, any device)."""
    t = qkv.shape[0]
    pos = _positions(t, seq_len, qkv.device, pos_ids)
    x = qkv.view(t, hq + 2 * hkv, hd)
    qk = x[:, : hq + hkv]
    if rot_dim < hd:
        rot = reference.rope_reference(qk[..., :rot_dim], pos, base, scale, offset, interleaved, inverse)
        qk = torch.cat([rot, qk[..., rot_dim:]], dim=-1)
    else:
        qk = reference.rope_reference(qk, pos, base, scale, offset, interleaved, inverse)
    return torch.cat([qk, x[:, hq + hkv:]], dim=1).reshape(t, -1)


class _RopeAttention(torch.autograd.Function):
    """RoPE (in place on the packed projection output) + causal flash attention."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, hd, seq_len, rope, cu_seqlens, causal, scale, rot_dim=None, dropout_p=0.0):
        from . import attention as attn

        t = qkv.shape[0]
        rot_dim = hd if rot_dim is None else rot_dim
        if rope is not None:
            base, rscale, offset, interleaved, pos_ids = rope
            kernels.rope(qkv, qkv, nheads=hq + hkv, head_dim=hd, tokens=t, seq_len=seq_len, base=base, scale=rscale,
                         offset=offset, interleaved=interleaved, pos_ids=pos_ids, row_stride=qkv.stride(0),
                         out_stride=qkv.stride(0), rot_dim=rot_dim)
        seed = attn.next_dropout_seed(qkv.device) if dropout_p > 0 else None
        out, lse = attn.flash_fwd(qkv, hq, hkv, hd, seq_len, cu_seqlens=cu_seqlens, causal=causal, scale=scale,
                                  dropout_p=dropout_p, dropout_seed=seed)
        ctx.save_for_backward(qkv, out, lse, cu_seqlens if cu_seqlens is not None else lse,
                              seed if seed is not None else lse)
        ctx.meta = (hq, hkv, hd, seq_len, rope, cu_seqlens is not None, causal, scale, rot_dim, dropout_p)
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import attention as attn

        qkv, out, lse, cu, seed = ctx.saved_tensors
        hq, hkv, hd, seq_len, rope, has_cu, causal, scale, rot_dim, dropout_p = ctx.meta
        dqkv = attn.flash_bwd(dout.contiguous(), qkv, out, lse, hq, hkv, hd, seq_len,
                              cu_seqlens=cu if has_cu else None, causal=causal, scale=scale, dropout_p=dropout_p,
                              dropout_seed=seed if dropout_p > 0 else None)
        if rope is not None:
            base, rscale, offset, interleaved, pos_ids = rope
            kernels.rope(dqkv, dqkv, nheads=hq + hkv, head_dim=hd, tokens=dqkv.shape[0], seq_len=seq_len, base=base,
                         scale=rscale, offset=offset, interleaved=interleaved, inverse=True, pos_ids=pos_ids,
                         row_stride=dqkv.stride(0), out_stride=dqkv.stride(0), rot_dim=rot_dim)
        return dqkv, None, None, None, None, None, None, None, None, None, None


def rope_attention(qkv: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, seq_len: int,
                   rope: Optional[tuple] = None, rot_dim: Optional[int] = None, causal: bool = True,
                   scale: Optional[float] = None, cu_seqlens: Optional[torch.Tensor] = None,
                   attn_mask: Optional[torch.Tensor] = None, dropout_p: float = 0.0, fused: bool = True,
                   training: bool = False) -> torch.Tensor:
    """Self attention on a packed projection ``qkv`` [T, (Hq + 2 Hkv) * hd] (T = batch * seq_len,
    batch-major). ``rope`` = (base, scale, offset, interleaved, pos_ids or None). Returns [T, Hq*hd].

    ``fused`` selects the flash kernel (causal or full, document boundaries via cu_seqlens, partial rotary and
    attention dropout inside the kernel); scores are materialised only for an arbitrary boolean mask, for head
    sizes other than 64 / 128, on CPU and in fp32."""
    t = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    rot_dim = head_dim if rot_dim is None else rot_dim
    native_ok = (use_native(qkv) and fused and head_dim in (64, 128) and rot_dim % 2 == 0 and 0 < rot_dim <= head_dim
                 and attn_mask is None)
    if native_ok:
        from . import attention as attn

        if attn.available():
            q = qkv if qkv.is_contiguous() else qkv.contiguous()
            return _RopeAttention.apply(q, num_heads, num_kv_heads, head_dim, seq_len, rope, cu_seqlens, causal,
                                        scale, rot_dim, float(dropout_p) if training else 0.0)
    if attn_mask is not None:
        note_fallback("attention", "an explicit boolean mask materialises the scores (document boundaries go "
                                   "through cu_seqlens on the flash kernel)", qkv)
    elif fused:
        note_fallback("attention", f"head size {head_dim} (rotary width {rot_dim}) is outside the flash kernel's "
                                   "64 / 128", qkv)
    if rope is not None:
        base, rscale, offset, interleaved, pos_ids = rope
        qkv = rope_reference_packed(qkv, num_heads, num_kv_heads, head_dim, seq_len, base, rscale, offset,
                                    interleaved, rot_dim, pos_ids)
    b = t // seq_len
    x = qkv.view(b, seq_len, num_heads + 2 * num_kv_heads, head_dim)
    q, k, v = x[:, :, :num_heads], x[:, :, num_heads:num_heads + num_kv_heads], x[:, :, num_heads + num_kv_heads:]
    mask = attn_mask
    if cu_seqlens is not None and mask is None:
        mask = document_mask(cu_seqlens, b, seq_len, qkv.device)
    out = _materialised_attention(q, k, v, causal, scale, mask, dropout_p if training else 0.0)
    return out.reshape(t, num_heads * head_dim)


def document_mask(cu_seqlens: torch.Tensor, b: int, s: int, device) -> torch.Tensor:
    """Boolean [B,1,S,S] mask allowing attention only inside a document; cu_seqlens index the flat
    batch-major token stream."""
    tok = torch.arange(b * s, device=device)
    doc = torch.bucketize(tok, cu_seqlens[1:].to(device), right=True).view(b, s)
    return (doc[:, :, None] == doc[:, None, :]).unsqueeze(1)


def _materialised_attention(q, k, v, causal, scale, mask, dropout_p):
    b, s, hq, hd = q.shape
    hkv = k.shape[2]
    qf, kf, vf = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if hkv != hq:
        kf = kf.repeat_interleave(hq // hkv, dim=1)
        vf = vf.repeat_interleave(hq // hkv, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)).float() * scale
    if causal:
        cm = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
        scores = scores.masked_fill(~cm, float("-inf"))
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    p = torch.softmax(scores, dim=-1).to(q.dtype)
    if dropout_p > 0:
        p = F.dropout(p, dropout_p)
    out = torch.matmul(p, vf)
    return out.transpose(1, 2)
