"""Tensor-level wrappers around the native sm_100a kernels.

Each function validates shapes/strides, allocates outputs with torch (so the
caching allocator and stream semantics stay PyTorch's) and launches the kernel on
the current CUDA stream. These wrappers have no autograd; see
:mod:`ironcore_b200.ops.functional` for differentiable ops.
"""

from __future__ import annotations


from typing import Optional

import torch

from . import native
from .native import call, dtype_code, ptr, query, stream_ptr

ACT_KINDS = {"relu": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "sigmoid": 4}
# gated activations: name -> (kind, gate_is_act). y = act(f) * g, or f * act(g) when gate_is_act.
GLU_KINDS = {
    "swiglu": (3, 0),
    "geglu": (2, 0),
    "geglu_erf": (1, 0),
    "reglu": (0, 0),
    "glu": (4, 1),
}


def _check_2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with a contiguous last dim, got shape {tuple(t.shape)} strides {t.stride()}")
    if (t.stride(0) * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: row pitch and base address must be multiples of 16 bytes")


native.register("icb_gemm_2sm", [native.P] * 5 + [native.I] * 3 + [native.L] * 4 + [native.I] * 4 + [native.P] * 2)

# Which plain (ungrouped) problems run on the CTA-pair kernel (256 x 256 tiles, tcgen05.mma.cta_group::2):
# "off" none, "on" all, "auto" those for which ``_two_sm_wins`` says so. Set by ``set_gemm_policy``.
_TWO_SM_POLICY = "auto"


def set_gemm_policy(two_sm: str) -> None:
    global _TWO_SM_POLICY
    if two_sm not in ("off", "on", "auto"):
        raise ValueError("two_sm policy must be off, on or auto")
    _TWO_SM_POLICY = two_sm


def two_sm_available() -> bool:
    lib = native.load()
    return lib is not None and hasattr(lib, "icb_gemm_2sm")


native.register("icb_cast_add", [native.P, native.P, native.P, native.L, native.I, native.L, native.L, native.I, native.P])
native.register("icb_gemm_splitk", [native.P] * 5 + [native.I] * 3 + [native.L] * 4 + [native.I] * 4 + [native.P] * 2)
_NUM_SMS = None


def _split_k_for(m: int, n: int, k: int) -> int:
    """How many CTAs share one output tile along K. Only problems with a few token rows against a wide
    weight matrix (decode steps) qualify: their 128 x 256 output tiles number far fewer than the SMs, so
    without the split a handful of CTAs would stream the whole weight matrix."""
    global _NUM_SMS
    if m > 256 or k < 512:
        return 1
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    if tiles * 2 > _NUM_SMS:
        return 1
    return max(1, min(_NUM_SMS // tiles, k // 256, 32))


def _accumulate_split(m: int, n: int, k: int) -> int:
    """Split of the K range for C += A B with an fp32 C (weight gradients accumulated in place); 1 = none.

    The partial products of the K ranges are added into C by TMA reduce-adds, which is what the product does
    anyway, so the split costs no workspace and no closing pass. It pays when whole-K tiles fill the machine
    badly: an 8-way tensor-parallel shard of a weight gradient (4096 x 1536, K = 4096 tokens) is 96 CTA-pair
    tiles on 74 pairs, two waves with the second a third full. Cost model, fitted to CUDA-event timings of the
    Llama-7B weight-gradient shards on B200 (within 5 % of the best measured choice on 10 of 11 shapes):
    waves x (k-blocks per work item + 12 k-block times of prologue / epilogue); CTA-pair tiles, which cannot
    split, cost 0.92 of that per wave. Measured: 4096 x 1536: 0.070 -> 0.059 ms; 512 x 4096: 0.043 -> 0.029 ms;
    1376 x 4096: 0.068 -> 0.059 ms; the 4-way shards and larger stay on CTA pairs."""
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    sms = _NUM_SMS
    kb = (k + 63) // 64
    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    if _two_sm_wins(m, n, k):
        pairs = ((m + 255) // 256) * ((n + 255) // 256)
        best_cost = -(-pairs // max(sms // 2, 1)) * (kb + 12.0) * 0.92
    else:
        best_cost = -(-tiles // sms) * (kb + 12.0)
    best = 1
    for s in (2, 3, 4):
        if kb // s < 8:
            break
        cost = -(-(tiles * s) // sms) * (-(-kb // s) + 12.0)
        if cost < best_cost:
            best, best_cost = s, cost
    return best


def _two_sm_wins(m: int, n: int, k: int) -> bool:
    """Measured on B200 (CUDA events, L2 flushed, bf16): the pair kernel is 1.03-1.23x faster than the
    single-CTA kernel on every Llama-7B layer shape, forward, dgrad and wgrad, including the 8-way
    tensor-parallel shards (4096 x 1536 x 4096, 4096 x 4096 x 1376): each CTA stages 32 KiB per k-block
    instead of 48 KiB for the same MMA work. Below a couple of 256 x 256 tiles per dimension the single-CTA
    kernel's finer tiling fills the machine better."""
    return m >= 512 and n >= 512 and k >= 128


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_major: int,
    b_major: int,
    m: int,
    n: int,
    k: int,
    out: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    group_mode: int = 0,
    num_groups: int = 1,
    group_table: Optional[torch.Tensor] = None,
    b_group_stride: int = 0,
    max_ctas: int = 0,
    two_sm: Optional[bool] = None,
) -> torch.Tensor:
    """C[m,n] = A*B (+bias) (+residual) on the tcgen05 GEMM.

    a_major 0: ``a`` is [m, k] (k contiguous); 1: ``a`` is [k, m] (m contiguous).
    b_major 0: ``b`` is [n, k] (k contiguous); 1: ``b`` is [k, n] (n contiguous).
    ``residual`` must have the output dtype and may alias ``out`` (accumulation).
    ``two_sm``: run on CTA pairs (None = the policy set with ``set_gemm_policy``).
    """
    in_dt = a.dtype
    if b.dtype != in_dt or in_dt not in (torch.bfloat16, torch.float16):
        raise TypeError("gemm operands must both be bf16 or both fp16")
    out_dtype = out_dtype or (out.dtype if out is not None else in_dt)
    if out_dtype not in (in_dt, torch.float32):
        raise TypeError("gemm output must be the input dtype or fp32")
    if group_mode == 2:
        out_shape = (num_groups, m, n)
    else:
        out_shape = (m, n)
    if out is None:
        out = torch.empty(out_shape, dtype=out_dtype, device=a.device)
    ldc = out.stride(-2)
    if out.stride(-1) != 1 or (ldc * out.element_size()) % 16 or out.data_ptr() % 16:
        raise ValueError("gemm output must be row-major with 16-byte aligned rows")
    _check_2d(a if a.dim() == 2 else a.reshape(-1, a.shape[-1]), "a")
    lda = a.stride(-2)
    ldb = b.stride(-2)
    if b.stride(-1) != 1 or (ldb * 2) % 16 or b.data_ptr() % 16:
        raise ValueError("gemm operand b must be row-major with 16-byte aligned rows")
    ldr = 0
    if residual is not None:
        if residual.dtype != out_dtype or residual.stride(-1) != 1:
            raise ValueError("residual must match the output dtype and be row-major")
        ldr = residual.stride(-2)
    if bias is not None and bias.dtype != in_dt:
        bias = bias.to(in_dt)
    if group_table is not None and group_table.dtype != torch.int32:
        raise TypeError("group_table must be int32")
    if group_mode == 0 and max_ctas == 0 and residual is not out and a.is_cuda:
        split = _split_k_for(m, n, k)
        if split > 1:
            ws = torch.zeros((m, n), dtype=torch.float32, device=a.device)
            call("icb_gemm_splitk", ptr(a), ptr(b), ptr(ws), ptr(bias), None, int(m), int(n), int(k), int(lda),
                 int(ldb), int(ws.stride(0)), 0, int(a_major), int(b_major), dtype_code(in_dt), int(split),
                 ptr(native.status_tensor(a.device)), stream_ptr())
            if n % 8 == 0 and out.dtype == in_dt and (residual is None or residual.dtype == in_dt):
                call("icb_cast_add", ptr(ws), ptr(residual), ptr(out), int(m), int(n), int(ldr), int(ldc),
                     dtype_code(in_dt), stream_ptr())
            else:
                if residual is not None:
                    ws += residual
                out.copy_(ws)
            return out
    if (group_mode == 0 and max_ctas == 0 and residual is out and out_dtype == torch.float32 and bias is None
            and two_sm is None and a.is_cuda and n % 4 == 0):
        split = _accumulate_split(m, n, k)
        if split > 1:
            call("icb_gemm_splitk", ptr(a), ptr(b), ptr(out), None, None, int(m), int(n), int(k), int(lda), int(ldb),
                 int(ldc), 0, int(a_major), int(b_major), dtype_code(in_dt), int(split),
                 ptr(native.status_tensor(a.device)), stream_ptr())
            return out
    if two_sm is None:
        two_sm = _TWO_SM_POLICY == "on" or (_TWO_SM_POLICY == "auto" and _two_sm_wins(m, n, k))
    if group_mode == 0 and two_sm and max_ctas == 0:
        call("icb_gemm_2sm", ptr(a), ptr(b), ptr(out), ptr(bias), ptr(residual), int(m), int(n), int(k), int(lda),
             int(ldb), int(ldc), int(ldr), int(a_major), int(b_major), dtype_code(in_dt),
             1 if out_dtype == torch.float32 else 0, ptr(native.status_tensor(a.device)), stream_ptr())
        return out
    call(
        "icb_gemm",
        ptr(a), ptr(b), ptr(out), ptr(bias), ptr(residual),
        int(m), int(n), int(k), int(lda), int(ldb), int(ldc), int(ldr),
        int(a_major), int(b_major), dtype_code(in_dt), 1 if out_dtype == torch.float32 and in_dt != torch.float32 else 0,
        int(group_mode), int(num_groups), ptr(group_table), int(b_group_stride),
        ptr(native.status_tensor(a.device)), int(max_ctas), stream_ptr(),
    )
    return out


def mm_nn(x: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """x[M,K] @ w[K,N] (weights stored [in, out])."""
    return gemm(x, w, a_major=0, b_major=1, m=x.shape[0], n=w.shape[1], k=x.shape[1], **kw)


def mm_nt(dy: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """dy[M,N] @ w[K,N]^T -> [M,K]."""
    return gemm(dy, w, a_major=0, b_major=0, m=dy.shape[0], n=w.shape[0], k=dy.shape[1], **kw)


def mm_tn(x: torch.Tensor, dy: torch.Tensor, **kw) -> torch.Tensor:
    """x[M,K]^T @ dy[M,N] -> [K,N]."""
    return gemm(x, dy, a_major=1, b_major=1, m=x.shape[1], n=dy.shape[1], k=x.shape[0], **kw)


# ---------------------------------------------------------------------------
# normalisation
# ---------------------------------------------------------------------------
def norm_fwd(x, weight, bias, eps: float, rms: bool, residual=None, w_offset: float = 0.0, store_sum: bool = True,
             out=None):
    """Returns (y, h, mean, rstd). ``h`` is x+residual (or x itself when no residual). ``out``: contiguous
    tensor of x's shape and dtype that receives ``y`` (e.g. this rank's rows of a gather buffer)."""
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    m = x2.shape[0]
    if out is not None and (out.shape != x2.shape or out.dtype != x2.dtype or not out.is_contiguous()):
        raise ValueError("norm_fwd: `out` must be a contiguous tensor of the input's 2-D shape and dtype")
    y = out if out is not None else torch.empty_like(x2)
    rstd = torch.empty(m, dtype=torch.float32, device=x.device)
    mean = None if rms else torch.empty(m, dtype=torch.float32, device=x.device)
    h = None
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, d)
        h = torch.empty_like(x2) if store_sum else None
    call(
        "icb_norm_fwd", ptr(x2), ptr(r2), ptr(weight), ptr(bias), ptr(y), ptr(h), ptr(mean), ptr(rstd),
        m, d, float(eps), float(w_offset), 1 if rms else 0, dtype_code(x.dtype), stream_ptr(),
        ptr(native.status_tensor(x.device)),
    )
    return y.view(x.shape), (h.view(x.shape) if h is not None else x), mean, rstd


def norm_bwd(dy, x, weight, mean, rstd, rms: bool, has_bias: bool, dres_in=None, w_offset: float = 0.0):
    """Returns (dx, dw, db). dres_in (optional) is added into dx inside the kernel."""
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    dy2 = dy.reshape(-1, d)
    m = x2.shape[0]
    parts = query("icb_norm_bwd_parts", m)
    scratch = torch.empty((2 if has_bias else 1) * parts * d, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x2)
    dw = torch.empty(d, dtype=torch.float32, device=x.device)
    db = torch.empty(d, dtype=torch.float32, device=x.device) if has_bias else None
    dr2 = dres_in.reshape(-1, d) if dres_in is not None else None
    call(
        "icb_norm_bwd", ptr(dy2), ptr(x2), ptr(weight), ptr(mean), ptr(rstd), ptr(dr2), ptr(dx), ptr(dw), ptr(db),
        ptr(scratch), m, d, float(w_offset), 1 if rms else 0, dtype_code(x.dtype), 1, 0, stream_ptr(),
        ptr(native.status_tensor(x.device)),
    )
    return dx.view(x.shape), dw, db


# ---------------------------------------------------------------------------
# rotary embedding
# ---------------------------------------------------------------------------
def rope(x: torch.Tensor, out: torch.Tensor, *, nheads: int, head_dim: int, tokens: int, seq_len: int,
         base: float, scale: float = 1.0, offset: int = 0, interleaved: bool = True, inverse: bool = False,
         pos_ids: Optional[torch.Tensor] = None, row_stride: Optional[int] = None,
         out_stride: Optional[int] = None, rot_dim: Optional[int] = None) -> torch.Tensor:
    """Rotate ``nheads`` heads starting at x's data pointer in rows of pitch ``row_stride`` elements.
    ``rot_dim`` < ``head_dim`` (partial rotary, in place only) rotates the first ``rot_dim`` elements of each head."""
    rs = row_stride if row_stride is not None else nheads * head_dim
    os_ = out_stride if out_stride is not None else rs
    call(
        "icb_rope", ptr(x), ptr(out), ptr(pos_ids), int(tokens), int(nheads), int(head_dim), int(rs), int(os_),
        int(seq_len), float(base), float(scale), int(offset), 1 if interleaved else 0, 1 if inverse else 0,
        dtype_code(x.dtype), stream_ptr(), int(rot_dim or head_dim),
    )
    return out


# ---------------------------------------------------------------------------
# activations
# ---------------------------------------------------------------------------
def glu_fwd(x: torch.Tensor, name: str, row_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``row_limit`` (int32 device tensor, one element): rows from that index on are not read and come out as
    zeros (the unused capacity of a padded expert layout, which no kernel has written)."""
    kind, gate_is_act = GLU_KINDS[name]
    f = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * f)
    y = torch.empty((x2.shape[0], f), dtype=x.dtype, device=x.device)
    call("icb_glu_fwd", ptr(x2), ptr(y), x2.shape[0], f, kind, gate_is_act, dtype_code(x.dtype), stream_ptr(),
         ptr(row_limit))
    return y.view(*x.shape[:-1], f)


def glu_bwd(dy: torch.Tensor, x: torch.Tensor, name: str, row_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
    kind, gate_is_act = GLU_KINDS[name]
    f = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * f)
    dy2 = dy.reshape(-1, f)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    dx = torch.empty_like(x2)
    call("icb_glu_bwd", ptr(dy2), ptr(x2), ptr(dx), x2.shape[0], f, kind, gate_is_act, dtype_code(x.dtype), stream_ptr(),
         ptr(row_limit))
    return dx.view(x.shape)


def act_fwd(x: torch.Tensor, name: str) -> torch.Tensor:
    xc = x.contiguous()
    y = torch.empty_like(xc)
    call("icb_act_fwd", ptr(xc), ptr(y), xc.numel(), ACT_KINDS[name], dtype_code(x.dtype), stream_ptr())
    return y


def act_bwd(dy: torch.Tensor, x: torch.Tensor, name: str) -> torch.Tensor:
    xc = x.contiguous()
    dyc = dy.contiguous()
    dx = torch.empty_like(xc)
    call("icb_act_bwd", ptr(dyc), ptr(xc), ptr(dx), xc.numel(), ACT_KINDS[name], dtype_code(x.dtype), stream_ptr())
    return dx


# ---------------------------------------------------------------------------
# embedding
# ---------------------------------------------------------------------------
def embedding_fwd(ids: torch.Tensor, weight: torch.Tensor, *, vocab_start: int = 0,
                  pos_table: Optional[torch.Tensor] = None, pos_ids: Optional[torch.Tensor] = None,
                  seq_len: int = 1) -> torch.Tensor:
    flat = ids.reshape(-1)
    if flat.dtype != torch.int64:
        flat = flat.long()
    t = flat.numel()
    d = weight.shape[1]
    out = torch.empty((t, d), dtype=weight.dtype, device=weight.device)
    call(
        "icb_embedding_fwd", ptr(flat), ptr(weight), ptr(pos_table), ptr(pos_ids), ptr(out), t, d, int(vocab_start),
        weight.shape[0], int(seq_len), dtype_code(weight.dtype), stream_ptr(),
    )
    return out.view(*ids.shape, d)


def embedding_bwd(rows: torch.Tensor, dy: torch.Tensor, num_rows: int, *, row_start: int = 0,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dW[rows[t] - row_start] += dy[t] (fp32 atomics). ``out`` (fp32 [num_rows, d]) is accumulated into."""
    flat = rows.reshape(-1)
    if flat.dtype != torch.int64:
        flat = flat.long()
    d = dy.shape[-1]
    dy2 = dy.reshape(-1, d).contiguous()
    dw = out if out is not None else torch.zeros((num_rows, d), dtype=torch.float32, device=dy.device)
    call("icb_embedding_bwd", ptr(flat), ptr(dy2), ptr(dw), flat.numel(), d, int(row_start), num_rows,
         dtype_code(dy.dtype), stream_ptr())
    return dw


# ---------------------------------------------------------------------------
# cross entropy
# ---------------------------------------------------------------------------
def ce_stats(logits: torch.Tensor, targets: torch.Tensor, *, vocab_start: int = 0, vocab_valid: Optional[int] = None):
    t, v = logits.shape
    vv = v if vocab_valid is None else vocab_valid
    rmax = torch.empty(t, dtype=torch.float32, device=logits.device)
    rsum = torch.empty_like(rmax)
    rtgt = torch.empty_like(rmax)
    call("icb_ce_stats", ptr(logits), ptr(targets), ptr(rmax), ptr(rsum), ptr(rtgt), t, v, logits.stride(0),
         int(vocab_start), int(vv), dtype_code(logits.dtype), stream_ptr())
    return rmax, rsum, rtgt


def ce_grad_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, gscale: torch.Tensor, *,
             vocab_start: int = 0, vocab_valid: Optional[int] = None) -> torch.Tensor:
    t, v = logits.shape
    vv = v if vocab_valid is None else vocab_valid
    call("icb_ce_grad", ptr(logits), ptr(targets), ptr(lse), ptr(gscale), t, v, logits.stride(0), int(vocab_start),
         int(vv), dtype_code(logits.dtype), stream_ptr())
    return logits


# ---------------------------------------------------------------------------
# optimizer helpers
# ---------------------------------------------------------------------------
def adam_step_(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, grad_scale_dev=None):
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    step_size = lr * (bc2 ** 0.5) / bc1
    call("icb_adam", ptr(p), ptr(g), ptr(m), ptr(v), p.numel(), float(lr), float(beta1), float(beta2), float(eps),
         float(weight_decay), float(step_size), float(grad_scale), ptr(grad_scale_dev), dtype_code(p.dtype),
         dtype_code(g.dtype), stream_ptr())


def sumsq(g: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[0] (+)= sum(g^2) on device; ``out`` is a 1-element fp32 tensor."""
    n = g.numel()
    parts = query("icb_sumsq_parts", n)
    scratch = torch.empty(parts, dtype=torch.float32, device=g.device)
    call("icb_sumsq", ptr(g), n, ptr(scratch), ptr(out), 1 if accumulate else 0, dtype_code(g.dtype), stream_ptr())
    return out


def clip_coef(total_sq: torch.Tensor, clip: float):
    norm = torch.empty(1, dtype=torch.float32, device=total_sq.device)
    coef = torch.empty(1, dtype=torch.float32, device=total_sq.device)
    call("icb_clip_coef", ptr(total_sq), float(clip), ptr(norm), ptr(coef), stream_ptr())
    return norm, coef
