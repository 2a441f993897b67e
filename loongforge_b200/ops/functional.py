"""Differentiable front-ends of the hot ops.

Each op has two implementations with identical semantics:
  * CUDA tensors -> the hand-written sm_100a kernels of ``csrc/`` (the extension is REQUIRED on
    a GPU machine; there is no silent fallback),
  * CPU tensors  -> a plain PyTorch expression, which is also the numerical oracle of the
    kernel tests.

Weight gradients follow Megatron's "gradient accumulation fusion": when a parameter carries a
fp32 ``main_grad`` buffer the wgrad GEMM accumulates straight into it from its TMEM epilogue
and autograd receives no gradient tensor for that parameter; ``param.grad_ready()`` (if set) is
called so that the data-parallel reducer can start on the bucket. Parameters used by any other
op receive ordinary autograd gradients, which the data-parallel wrapper folds into ``main_grad``
with a post-accumulate hook.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _ext

# ----------------------------------------------------------------------------- helpers


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda


def _C():
    return _ext.require()


def use_native_gemm(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    out: Optional[torch.Tensor] = None,
    out_mode: int = 0,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    alpha: float = 1.0,
    max_ctas: int = 0,
) -> torch.Tensor:
    """D = op(A) @ op(B)^T-style product on the tcgen05 GEMM (see csrc/gemm_sm100.h).

    K-major A is ``[M, K]``, MN-major A is ``[K, M]``; K-major B is ``[N, K]``, MN-major B is
    ``[K, N]``. ``out_mode``: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate into ``out``.
    """
    if a.is_cuda and _gemm_native_ok(a, b, a_mn_major, b_mn_major, out, bias, residual):
        return _C().gemm(a, b, out, a_mn_major, b_mn_major, out_mode, bias, residual, alpha,
                         _ext.status_tensor(a.device), max_ctas)
    # CPU, or a shape / dtype the tcgen05 GEMM does not take (an output narrower than 8 columns, fp32 operands):
    # the same contract in PyTorch math
    am = a.t() if a_mn_major else a
    bm = b if b_mn_major else b.t()
    d = (am.float() @ bm.float()) * alpha
    if bias is not None:
        d = d + bias.float()
    if residual is not None:
        d = d + residual.float()
    if out_mode == 0:
        d = d.to(a.dtype)
        if out is not None:
            out.copy_(d)
            return out
        return d
    if out_mode == 2:
        out.add_(d)
        return out
    if out is not None:
        out.copy_(d)
        return out
    return d


def _gemm_native_ok(a, b, a_mn, b_mn, out, bias, residual) -> bool:
    """Operands the tcgen05 GEMM accepts: bf16, unit inner stride, leading dimensions that are multiples of 8
    elements (16-byte rows for TMA and the vectorised epilogue), 16-byte aligned bases."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.dim() != 2 or b.dim() != 2:
        return False
    n = b.shape[1] if b_mn else b.shape[0]
    if n % 8 != 0:
        return False  # the output's leading dimension
    for t in (a, b, out, residual):
        if t is not None and (t.stride(-1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0):
            return False
    return bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous())


def grouped_gemm(a: torch.Tensor, x: Optional[torch.Tensor], weights, outs, tokens_per_expert, *, mode: int,
                 out_mode: int = 0) -> None:
    """One grouped tcgen05 launch over all experts (csrc/grouped_gemm_sm100.h): mode 0 forward,
    1 dgrad, 2 wgrad (``outs`` = one [N, K] tensor per expert; ``out_mode`` 2 accumulates in fp32)."""
    _C().grouped_gemm(a, x, list(weights), list(outs), [int(n) for n in tokens_per_expert], mode, out_mode,
                      _ext.status_tensor(a.device))


def _ld_ok(*ts: torch.Tensor) -> bool:
    for t in ts:
        if t.stride(-1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
            return False
    return True


# ----------------------------------------------------------------------------- linear


class _LinearFn(torch.autograd.Function):
    """y = x @ W^T (+ bias) (+ residual), W is [out, in] (forward / dgrad / wgrad on the tcgen05 GEMM)."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        res2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        y = gemm(x2, weight, bias=bias, residual=res2)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.in_shape = shp
        if len(shp) == 2:
            return y  # not a view: callers may rotate it in place (RoPE on the packed QKV)
        return y.reshape(*shp[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, weight.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn_major=True).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy2, x2, weight)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor):
    """dW = dy^T @ x. Accumulates into ``weight.main_grad`` when present (returns None then)."""
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=main_grad, out_mode=2)
        weight.grad_added_to_main_grad = True
        hook = getattr(weight, "grad_ready", None)
        if hook is not None:
            hook()
        return None
    return gemm(dy2, x2, a_mn_major=True, b_mn_major=True)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if use_native_gemm(x) and _ld_ok(weight) and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
        if not x.is_contiguous():
            x = x.contiguous()
        return _LinearFn.apply(x, weight, bias, residual)
    if getattr(weight, "main_grad", None) is not None:
        # CPU / odd-shape path still honours gradient-accumulation fusion.
        return _LinearFn.apply(x, weight, bias, residual)
    y = F.linear(x, weight, bias)
    return y + residual if residual is not None else y


# ----------------------------------------------------------------------------- RMSNorm


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * r * (w.float() + w_offset)).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, w_offset):
        xc = x.contiguous()
        y, rstd = _C().rmsnorm_fwd(xc, w, eps, w_offset)
        ctx.save_for_backward(xc, w, rstd)
        ctx.w_offset = w_offset
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _C().rmsnorm_bwd(dy.contiguous(), x, w, rstd, None, ctx.w_offset)
        return dx, dw.to(w.dtype), None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5, w_offset: float = 0.0) -> torch.Tensor:
    H = x.shape[-1]
    if _native(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and H % 8 == 0 and H <= 8192:
        return _RMSNormFn.apply(x, w, eps, w_offset)
    return rmsnorm_ref(x, w, eps, w_offset)


# ----------------------------------------------------------------------------- RoPE


def rope_freqs(positions: torch.Tensor, rot_dim: int, theta: float, scaling: float = 1.0) -> torch.Tensor:
    """Angles ``pos * theta^(-2i/rot_dim)`` as fp32 ``[len(positions), rot_dim/2]``."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=positions.device) / rot_dim))
    return torch.outer(positions.float() / scaling, inv).contiguous()


def rope_ref(x: torch.Tensor, freqs: torch.Tensor, rot_dim: int, rot_offset: int = 0, interleaved: bool = False,
             mscale: float = 1.0, sign: float = 1.0) -> torch.Tensor:
    """x [T, heads, D]; freqs [T, rot_dim/2] (already gathered per token)."""
    xf = x.float()
    cos = (freqs.cos() * mscale)[:, None, :]
    sin = (freqs.sin() * mscale * sign)[:, None, :]
    seg = xf[..., rot_offset:rot_offset + rot_dim]
    if interleaved:
        a, b = seg[..., 0::2], seg[..., 1::2]
        ra, rb = a * cos - b * sin, b * cos + a * sin
        rot = torch.stack([ra, rb], dim=-1).flatten(-2)
    else:
        h = rot_dim // 2
        a, b = seg[..., :h], seg[..., h:]
        rot = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    out = xf.clone()
    out[..., rot_offset:rot_offset + rot_dim] = rot
    return out.to(x.dtype)


class _RopeFn(torch.autograd.Function):
    """In-place rotation of selected heads of a packed ``[T, heads * D]`` (or ``[T, heads, D]``) tensor."""

    @staticmethod
    def forward(ctx, x, freqs, pos_ids, heads, D, rot_dim, rot_offset, group, rope_in_group, interleaved, mscale):
        T = x.shape[0]
        ctx.mark_dirty(x)
        _C().rope_(x, freqs, pos_ids, T, heads, D, rot_dim, rot_offset, x.stride(0), D, group,
                   rope_in_group, interleaved, mscale, 1.0)
        ctx.save_for_backward(freqs, pos_ids) if pos_ids is not None else ctx.save_for_backward(freqs)
        ctx.has_pos = pos_ids is not None
        ctx.cfg = (heads, D, rot_dim, rot_offset, group, rope_in_group, interleaved, mscale)
        return x

    @staticmethod
    def backward(ctx, dy):
        if ctx.has_pos:
            freqs, pos_ids = ctx.saved_tensors
        else:
            (freqs,) = ctx.saved_tensors
            pos_ids = None
        heads, D, rot_dim, rot_offset, group, rope_in_group, interleaved, mscale = ctx.cfg
        dx = dy.clone(memory_format=torch.contiguous_format)
        T = dx.shape[0]
        _C().rope_(dx, freqs, pos_ids, T, heads, D, rot_dim, rot_offset, dx.stride(0), D, group,
                   rope_in_group, interleaved, mscale, -1.0)
        return (dx,) + (None,) * 10


def rope(x: torch.Tensor, freqs: torch.Tensor, *, pos_ids: Optional[torch.Tensor] = None, rot_dim: Optional[int] = None,
         rot_offset: int = 0, group: int = 1, rope_in_group: int = 1, interleaved: bool = False,
         mscale: float = 1.0, inplace: bool = False, head_dim: Optional[int] = None) -> torch.Tensor:
    """Rotary embedding on ``x [T, heads, D]`` (or ``[T, heads * D]`` with ``head_dim=D``).

    Heads are grouped in runs of ``group``; the first ``rope_in_group`` heads of each run rotate
    (packed QKV: ``group = q_per_kv + 2``, ``rope_in_group = q_per_kv + 1``). ``freqs`` holds fp32
    angles ``[P, rot_dim/2]``; token t uses row ``pos_ids[t]`` (or row t).
    """
    shape = x.shape
    if head_dim is not None:
        D = head_dim
        Hh = x.shape[-1] // D
    else:
        Hh, D = x.shape[-2], x.shape[-1]
    T = x.shape[0]
    rot_dim = D - rot_offset if rot_dim is None else rot_dim
    if _native(x) and x.dtype == torch.bfloat16:
        if pos_ids is not None:
            pos_ids = pos_ids.to(torch.int32).contiguous()
        # The kernel works in place; `inplace=True` lets it reuse a buffer the caller owns
        # exclusively (e.g. the fresh output of the QKV GEMM).
        if inplace and x.dim() == 2 and x.is_contiguous():
            xin = x
        else:
            xin = x.reshape(T, Hh * D).clone(memory_format=torch.contiguous_format)
        out = _RopeFn.apply(xin, freqs.float().contiguous(), pos_ids, Hh, D, rot_dim, rot_offset, group,
                            rope_in_group, interleaved, mscale)
        return out.view(shape)
    x3 = x.reshape(T, Hh, D)
    f = freqs if pos_ids is None else freqs[pos_ids.long()]
    f = f[:T]
    if group == 1 or rope_in_group >= group:
        return rope_ref(x3, f, rot_dim, rot_offset, interleaved, mscale).reshape(shape)
    xg = x3.reshape(T, Hh // group, group, D)
    rot = rope_ref(xg[:, :, :rope_in_group].reshape(T, -1, D), f, rot_dim, rot_offset, interleaved, mscale)
    rot = rot.reshape(T, Hh // group, rope_in_group, D)
    return torch.cat([rot, xg[:, :, rope_in_group:]], dim=2).reshape(shape)


# ----------------------------------------------------------------------------- SwiGLU


def swiglu_ref(x: torch.Tensor) -> torch.Tensor:
    g, u = x.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return _C().swiglu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _C().swiglu_bwd(dy.contiguous(), x)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``x = [gate | up]`` on the last dimension."""
    if _native(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0:
        return _SwiGLUFn.apply(x)
    return swiglu_ref(x)


# ----------------------------------------------------------------------------- attention


def _seq_ids(T: int, cu, device):
    """(sequence id, position inside the sequence, sequence length) of each of T packed tokens."""
    idx = torch.arange(T, device=device)
    if cu is None:
        return torch.zeros_like(idx), idx, torch.full((1,), T, device=device, dtype=idx.dtype)
    cu = cu.to(device=device, dtype=idx.dtype)
    seg = torch.bucketize(idx, cu[1:], right=True).clamp_(max=cu.numel() - 2)
    return seg, idx - cu[seg], cu[1:] - cu[:-1]


def attention_ref(q, k, v, causal=True, scale=None, cu_seqlens=None, cu_seqlens_k=None, return_lse=False):
    """Naive softmax attention in fp32. q [Tq, Hq, D], k/v [Tk, Hkv, D] -> [Tq, Hq, Dv]. Query and key sides may have
    different lengths (per sequence when boundaries are given); the causal mask is aligned to the bottom right:
    query i of a sequence sees keys j <= i + (k_len - q_len). Rows that see no key return 0 (lse = -inf)."""
    Tq, Hq, D = q.shape
    Tk, Hkv, Dv = k.shape[0], k.shape[1], v.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, 0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, 0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    seg_q, pos_q, len_q = _seq_ids(Tq, cu_seqlens, q.device)
    seg_k, pos_k, len_k = _seq_ids(Tk, cu_seqlens_k if cu_seqlens_k is not None else
                                   (cu_seqlens if Tq == Tk else None), q.device)
    mask = seg_q[:, None] == seg_k[None, :]
    if causal:
        off = (len_k - len_q)[seg_q]
        mask &= pos_k[None, :] <= (pos_q + off)[:, None]
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.masked_fill(torch.isinf(lse), 0.0).unsqueeze(-1))
    o = torch.matmul(p, vf).transpose(0, 1).to(q.dtype).reshape(Tq, Hq, Dv)
    return (o, lse) if return_lse else o


class _AttnFn(torch.autograd.Function):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] (strided views allowed, D <= 128) -> o [Tq, Hq, D]; also returns the
    log-sum-exp [Hq, Tq] (not differentiable) so that partial results can be merged (context parallelism)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, scale, causal):
        Hkv = k.shape[1]
        q4 = q.unflatten(1, (Hkv, q.shape[1] // Hkv))
        o, lse = _C().attn_fwd(q4, k, v, cu_q, cu_k, scale, causal, _ext.status_tensor(q.device))
        ctx.save_for_backward(q, k, v, o, lse, *[c for c in (cu_q, cu_k) if c is not None])
        ctx.cfg = (scale, causal, cu_q is not None, cu_k is not None)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, *rest = ctx.saved_tensors
        scale, causal, has_q, has_k = ctx.cfg
        cu_q = rest[0] if has_q else None
        cu_k = rest[1] if has_k else None
        dq, dk, dv = attention_backward(do, q, k, v, o, lse, cu_q, cu_k, scale, causal)
        return dq, dk, dv, None, None, None, None


def attention_backward(do, q, k, v, o, lse, cu_q, cu_k, scale, causal):
    """Gradients of the native attention from a saved output and log-sum-exp. `o` / `lse` may be the MERGED result of
    several partial calls (ring / all-gather context parallelism): the probabilities are recomputed against the
    given lse, so the returned dk / dv are this key block's share."""
    if do.stride(2) != 1 or do.stride(1) % 8 or do.stride(0) % 8:
        do = do.contiguous()
    Hkv = k.shape[1]
    R = q.shape[1] // Hkv
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    _C().attn_bwd(do, q.unflatten(1, (Hkv, R)), k, v, o, lse, dq.unflatten(1, (Hkv, R)), dk, dv, cu_q, cu_k, scale,
                  causal, _ext.status_tensor(q.device))
    return dq, dk, dv


class _AttnPackedFn(torch.autograd.Function):
    """Attention straight on the packed QKV GEMM output ``[T, G*(R+2)*D]`` (Megatron's per-group
    ``[q_0..q_{R-1}, k, v]`` order): no split copies forward, and the backward kernels write dq,
    dk, dv into ONE packed gradient buffer that feeds the QKV dgrad/wgrad GEMMs directly."""

    @staticmethod
    def forward(ctx, qkv, G, R, cu_seqlens, scale, causal):
        T = qkv.shape[0]
        D = qkv.shape[1] // (G * (R + 2))
        pk = qkv.view(T, G, R + 2, D)
        o, lse = _C().attn_fwd(pk[:, :, :R], pk[:, :, R], pk[:, :, R + 1], cu_seqlens, None, scale, causal,
                               _ext.status_tensor(qkv.device))
        ctx.save_for_backward(qkv, o, lse, *([cu_seqlens] if cu_seqlens is not None else []))
        ctx.cfg = (G, R, D, scale, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, *rest = ctx.saved_tensors
        cu = rest[0] if rest else None
        G, R, D, scale, causal = ctx.cfg
        T = qkv.shape[0]
        if do.stride(2) != 1 or do.stride(1) % 8 or do.stride(0) % 8:
            do = do.contiguous()
        pk = qkv.view(T, G, R + 2, D)
        dqkv = torch.empty_like(qkv)
        dpk = dqkv.view(T, G, R + 2, D)
        _C().attn_bwd(do, pk[:, :, :R], pk[:, :, R], pk[:, :, R + 1], o, lse, dpk[:, :, :R], dpk[:, :, R],
                      dpk[:, :, R + 1], cu, None, scale, causal, _ext.status_tensor(qkv.device))
        return dqkv, None, None, None, None, None


_ATTN_IMPL = {"impl": "auto"}


def set_attention_impl(name: str) -> None:
    """'auto' (own kernel when compiled and shape supported), 'native', or 'sdpa' (library baseline)."""
    assert name in ("auto", "native", "sdpa")
    _ATTN_IMPL["impl"] = name


def native_attention_supported(q, k, v) -> bool:
    """The tcgen05 kernel covers bf16 with one head dim <= 128 (a multiple of 8) for q, k and v."""
    m = _ext.get()
    D = q.shape[-1]
    return (m is not None and hasattr(m, "attn_fwd") and q.is_cuda and q.dtype == torch.bfloat16
            and D <= 128 and D % 8 == 0 and k.shape[-1] == D and v.shape[-1] == D)


def attention_packed_supported(qkv: torch.Tensor, head_dim: int) -> bool:
    m = _ext.get()
    return (_ATTN_IMPL["impl"] != "sdpa" and m is not None and hasattr(m, "attn_fwd") and qkv.is_cuda
            and qkv.dtype == torch.bfloat16 and head_dim <= 128 and head_dim % 8 == 0 and qkv.dim() == 2
            and qkv.is_contiguous())


def attention_packed(qkv: torch.Tensor, groups: int, q_per_group: int, *, causal: bool = True,
                     scale: Optional[float] = None, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention on a packed ``[T, G*(R+2)*D]`` QKV buffer -> ``[T, G*R, D]``."""
    D = qkv.shape[1] // (groups * (q_per_group + 2))
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    cu = cu_seqlens.to(torch.int32).contiguous() if cu_seqlens is not None else None
    return _AttnPackedFn.apply(qkv, groups, q_per_group, cu, scale, causal)


def _strides_ok(t):
    return t.stride(2) == 1 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def attention_with_lse(q, k, v, *, causal=True, scale=None, cu_seqlens=None, cu_seqlens_k=None):
    """(output [Tq, Hq, D], log-sum-exp [Hq, Tq] fp32) of one attention call; the building block of the
    context-parallel schemes, which merge partial results by their log-sum-exp. Native kernel on a GPU, the fp32
    formulation elsewhere."""
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if q.is_cuda and _ATTN_IMPL["impl"] != "sdpa" and native_attention_supported(q, k, v):
        cq = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous() if cu_seqlens is not None else None
        ck = cu_seqlens_k.to(device=q.device, dtype=torch.int32).contiguous() if cu_seqlens_k is not None else None
        q, k, v = (t if _strides_ok(t) else t.contiguous() for t in (q, k, v))
        return _AttnFn.apply(q, k, v, cq, ck, scale, causal)
    return attention_ref(q, k, v, causal, scale, cu_seqlens, cu_seqlens_k, return_lse=True)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
              scale: Optional[float] = None, cu_seqlens: Optional[torch.Tensor] = None,
              cu_seqlens_k: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax attention over packed tokens. q [Tq, Hq, D], k/v [Tk, Hkv, D] -> [Tq, Hq, Dv]. With Tq != Tk the causal
    mask is aligned to the bottom right (per sequence when boundaries are given)."""
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    impl = _ATTN_IMPL["impl"]
    if q.is_cuda and impl != "sdpa" and native_attention_supported(q, k, v):
        return attention_with_lse(q, k, v, causal=causal, scale=scale, cu_seqlens=cu_seqlens,
                                  cu_seqlens_k=cu_seqlens_k)[0]
    if impl == "native" and q.is_cuda:
        raise RuntimeError("native attention requested but not available for this shape")
    same = q.shape[0] == k.shape[0] and cu_seqlens_k is None
    if q.is_cuda and cu_seqlens is None and same:
        Hq, Hkv = q.shape[1], k.shape[1]
        o = F.scaled_dot_product_attention(
            q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
            is_causal=causal, scale=scale, enable_gqa=Hq != Hkv)
        return o[0].transpose(0, 1).contiguous()
    if q.is_cuda and same:
        # library baseline for dtypes / head dims the tcgen05 kernel does not cover (fp32, head dim > 128):
        # block-diagonal (+ causal) mask from the sequence boundaries
        T = q.shape[0]
        idx = torch.arange(T, device=q.device)
        seg = torch.bucketize(idx, cu_seqlens[1:].to(q.device), right=True)
        mask = seg[:, None] == seg[None, :]
        if causal:
            mask &= idx[None, :] <= idx[:, None]
        Hq, Hkv = q.shape[1], k.shape[1]
        o = F.scaled_dot_product_attention(
            q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], attn_mask=mask[None, None],
            scale=scale, enable_gqa=Hq != Hkv)
        return o[0].transpose(0, 1).contiguous()
    return attention_ref(q, k, v, causal, scale, cu_seqlens, cu_seqlens_k)


# ----------------------------------------------------------------------------- fused linear + cross entropy


def _tp_allreduce(t: torch.Tensor, group, op):
    if group is not None and torch.distributed.get_world_size(group) > 1:
        torch.distributed.all_reduce(t, op=op, group=group)
    return t


class _LinearCEFn(torch.autograd.Function):
    """Token-chunked ``hidden @ W^T`` + softmax cross entropy that never holds ``[T, V]`` logits.

    Gradients w.r.t. hidden and W are produced in the forward pass (per chunk: logits GEMM ->
    row statistics -> TP all-reduce of max/sum/target -> in-place dlogits -> dgrad/wgrad GEMMs)
    and scaled by the incoming scalar gradient in backward. Matches the chunked algorithm of
    docs/source/features/fused_linear_cross_entropy.md:7-44 with vocabulary-parallel weights.
    """

    @staticmethod
    def forward(ctx, hidden, weight, labels, loss_mask, vocab_start, valid_v, tp_group, chunk_tokens, fused_scale):
        T, H = hidden.shape
        V = weight.shape[0]
        native = hidden.is_cuda and hidden.dtype == torch.bfloat16 and V % 8 == 0
        dev = hidden.device
        losses = torch.empty(T, dtype=torch.float32, device=dev)
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dh = torch.empty_like(hidden) if need_dh else None
        main_grad = getattr(weight, "main_grad", None)
        # Fast path: the caller told us the scalar the masked-sum loss will be multiplied with,
        # so dW goes straight into main_grad (no [V, H] temporary) and dh is final.
        fused = fused_scale is not None and main_grad is not None
        dw = None
        if need_dw:
            dw = main_grad.view(V, H) if fused else torch.zeros(V, H, dtype=torch.float32, device=dev)
        mask_f = loss_mask.float() if loss_mask is not None else torch.ones(T, dtype=torch.float32, device=dev)
        if fused_scale is not None:
            mask_f = mask_f * fused_scale
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            hc = hidden[s:e]
            lab = labels[s:e].contiguous()
            if native:
                logits = gemm(hc, weight)
                mx, sm, tg = _C().ce_stats(logits, lab, vocab_start, valid_v)
            else:
                logits = (hc.float() @ weight.float().t())
                lv = logits[:, :valid_v]
                mx = lv.max(dim=-1).values
                sm = torch.exp(lv - mx[:, None]).sum(-1)
                li = lab - vocab_start
                inr = (li >= 0) & (li < valid_v)
                tg = torch.where(inr, logits.gather(1, li.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(mx))
            gmax = _tp_allreduce(mx.clone(), tp_group, torch.distributed.ReduceOp.MAX)
            sm = sm * torch.exp(mx - gmax)
            packed = torch.stack([sm, tg])
            _tp_allreduce(packed, tp_group, torch.distributed.ReduceOp.SUM)
            gsum, gt = packed[0], packed[1]
            losses[s:e] = torch.log(gsum) + gmax - gt
            if need_dh or need_dw:
                sc = mask_f[s:e].contiguous()
                if native:
                    _C().ce_dlogits_(logits, lab, gmax, gsum.contiguous(), sc, vocab_start, valid_v)
                    dl = logits
                else:
                    p = torch.exp(logits - gmax[:, None]) / gsum[:, None]
                    p[:, valid_v:] = 0
                    li = lab - vocab_start
                    inr = (li >= 0) & (li < valid_v)
                    onehot = torch.zeros_like(p)
                    onehot.scatter_(1, li.clamp(0, V - 1)[:, None], inr.float()[:, None])
                    dl = ((p - onehot) * sc[:, None]).to(hidden.dtype)
                if need_dh:
                    gemm(dl, weight, b_mn_major=True, out=dh[s:e]) if native else dh[s:e].copy_(
                        (dl.float() @ weight.float()).to(hidden.dtype))
                if need_dw:
                    if native:
                        gemm(dl, hc, a_mn_major=True, b_mn_major=True, out=dw, out_mode=2)
                    else:
                        dw.add_(dl.float().t() @ hc.float())
        ctx.fused_scale = fused_scale
        ctx.fused = fused
        if fused and need_dw:
            weight.grad_added_to_main_grad = True
        ctx.save_for_backward(dh if dh is not None else torch.empty(0),
                              dw if (dw is not None and not fused) else torch.empty(0))
        ctx.weight = weight
        ctx.tp_group = tp_group
        return losses

    @staticmethod
    def backward(ctx, dlosses):
        # The per-token scaling was folded into the stored gradients through `loss_mask`;
        # the consumer reduces `losses * mask` with a scalar weight, so dlosses = c * mask.
        dh, dw = ctx.saved_tensors
        weight = ctx.weight
        if ctx.fused_scale is not None:
            # gradients were finalised in forward with the promised scale
            if ctx.fused:
                hook = getattr(weight, "grad_ready", None)
                if hook is not None:
                    hook()
                gw = None
            else:
                gw = dw.to(weight.dtype) if dw.numel() > 0 else None
            return (dh if dh.numel() > 0 else None), gw, None, None, None, None, None, None, None
        nz = dlosses[dlosses != 0]
        c = nz[0] if nz.numel() > 0 else dlosses.new_zeros(())
        gh = gw = None
        if dh.numel() > 0:
            gh = dh * c.to(dh.dtype)
        if dw.numel() > 0:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                main_grad.add_(dw.view_as(main_grad), alpha=float(c))
                weight.grad_added_to_main_grad = True
                hook = getattr(weight, "grad_ready", None)
                if hook is not None:
                    hook()
            else:
                gw = (dw * c).to(weight.dtype)
        return gh, gw, None, None, None, None, None, None, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         loss_mask: Optional[torch.Tensor] = None, *, vocab_start: int = 0,
                         valid_vocab: Optional[int] = None, tp_group=None, chunk_tokens: int = 2048,
                         fused_scale: Optional[float] = None) -> torch.Tensor:
    """Per-token CE losses ``[T]`` of ``softmax(hidden @ W^T)``; W is this rank's vocab slice.

    The caller must reduce the result as ``(losses * loss_mask).sum() * c`` for a scalar ``c``
    (the masked-sum loss of loongforge/train/get_loss_func.py:16-98); the gradients stored in
    the forward pass assume exactly that form. When the caller knows ``c`` up front it passes
    it as ``fused_scale``: the weight gradient then accumulates directly into ``weight.main_grad``
    from the wgrad GEMM epilogue and no ``[V, H]`` temporary exists.

    Under vocabulary parallelism the returned hidden gradient is this rank's PARTIAL sum; the
    mapping that brought `hidden` into the TP region (copy-to-TP or sequence-parallel gather)
    reduces it in its own backward.
    """
    valid_v = weight.shape[0] if valid_vocab is None else valid_vocab
    if not torch.is_grad_enabled():
        # the gradients are computed in the forward pass: make sure an evaluation-only call computes (and accumulates
        # into main_grad) none
        hidden, weight = hidden.detach(), weight.detach()
    return _LinearCEFn.apply(hidden, weight, labels, loss_mask, vocab_start, valid_v, tp_group, chunk_tokens,
                             fused_scale)


def cross_entropy_ref(hidden, weight, labels):
    logits = hidden.float() @ weight.float().t()
    return F.cross_entropy(logits, labels, reduction="none")


# ----------------------------------------------------------------------------- optimizer math


def adam_step(master, grad, exp_avg, exp_avg_sq, model_out, *, lr, beta1, beta2, eps, weight_decay, step,
              grad_scale=1.0):
    """AdamW on flat fp32 master weights (decoupled decay), optional bf16 model copy written in the same pass."""
    if master.is_cuda:
        _C().adam_step_(master, grad, exp_avg, exp_avg_sq, model_out, lr, beta1, beta2, eps, weight_decay, step,
                        grad_scale)
        return
    g = grad.float() * grad_scale
    m = exp_avg.float().mul_(beta1).add_(g, alpha=1 - beta1)
    v = exp_avg_sq.float().mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * master
    master.add_(upd, alpha=-lr)
    exp_avg.copy_(m)
    exp_avg_sq.copy_(v)
    if model_out is not None:
        model_out.copy_(master)


def sum_of_squares(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous():
        _C().sumsq_(x, out)
    else:
        out.add_(x.float().pow(2).sum())
    return out


# ----------------------------------------------------------------------------- fp32 master as (bf16, int16 remainder)


def master_join(w: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
    """Exact fp32 master weights from the bf16 weights and their int16 remainders."""
    if w.is_cuda:
        return _C().master_join(w.contiguous(), lo.contiguous())
    bits = (w.contiguous().view(torch.int16).to(torch.int32) << 16) + lo.to(torch.int32)
    return bits.view(torch.float32)


def master_split(master: torch.Tensor, w: torch.Tensor, lo: torch.Tensor, write_w: bool = True) -> None:
    """Split fp32 `master` into round-to-nearest bf16 `w` (optional) and the int16 remainder `lo`."""
    if master.is_cuda:
        _C().master_split_(master.contiguous(), w, lo, write_w)
        return
    wb = master.to(torch.bfloat16)
    hi = wb.view(torch.int16).to(torch.int32) << 16
    lo.copy_((master.contiguous().view(torch.int32) - hi).to(torch.int16))
    if write_w:
        w.copy_(wb)


def adam_step_remainder(w, lo, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step,
                        grad_scale=1.0):
    """AdamW where the fp32 master weight is the exact pair (bf16 `w`, int16 `lo`); updates both in place."""
    if w.is_cuda:
        _C().adam_step_remainder_(w, lo, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step,
                                  grad_scale)
        return
    master = master_join(w, lo).clone()
    adam_step(master, grad, exp_avg, exp_avg_sq, None, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
              weight_decay=weight_decay, step=step, grad_scale=grad_scale)
    master_split(master, w, lo, True)


# ----------------------------------------------------------------------------- memory-lean fused blocks


class _NormLinearFn(torch.autograd.Function):
    """y = RMSNorm(x; g) @ W^T (+ bias). Only x and rstd are kept; the normalised activations are
    recomputed in backward (one bandwidth-bound pass) instead of being stored."""

    @staticmethod
    def forward(ctx, x, ln_w, weight, bias, eps, w_offset):
        xn, rstd = _C().rmsnorm_fwd(x, ln_w, eps, w_offset)
        y = gemm(xn, weight, bias=bias)
        ctx.save_for_backward(x, ln_w, rstd, weight)
        ctx.cfg = (eps, w_offset, bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, ln_w, rstd, weight = ctx.saved_tensors
        eps, w_offset, has_bias = ctx.cfg
        dy = dy.contiguous()
        xn, _ = _C().rmsnorm_fwd(x, ln_w, eps, w_offset)
        dw = _wgrad(dy, xn, weight) if ctx.needs_input_grad[2] else None
        del xn
        dxn = gemm(dy, weight, b_mn_major=True)
        dx, dg = _C().rmsnorm_bwd(dxn, x, ln_w, rstd, None, w_offset)
        db = dy.float().sum(0).to(dy.dtype) if has_bias else None
        return dx, dg.to(ln_w.dtype), dw, db, None, None


def norm_linear_supported(x, ln_w, weight) -> bool:
    H = x.shape[-1]
    return (x.is_cuda and x.dim() == 2 and x.dtype == torch.bfloat16 and ln_w.dtype == torch.bfloat16
            and H % 8 == 0 and H <= 8192 and weight.shape[0] % 8 == 0 and _ld_ok(weight))


def norm_linear(x, ln_w, weight, bias=None, eps=1e-5, w_offset=0.0):
    return _NormLinearFn.apply(x.contiguous(), ln_w, weight, bias, eps, w_offset)


class _SwiGLULinearFn(torch.autograd.Function):
    """y = swiglu(h) @ W^T (+ residual). Keeps only h ([T, 2F]); silu(gate)*up is recomputed in backward."""

    @staticmethod
    def forward(ctx, h, weight, residual):
        a = _C().swiglu_fwd(h)
        y = gemm(a, weight, residual=residual)
        ctx.save_for_backward(h, weight)
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        h, weight = ctx.saved_tensors
        dy = dy.contiguous()
        a = _C().swiglu_fwd(h)
        dw = _wgrad(dy, a, weight) if ctx.needs_input_grad[1] else None
        del a
        da = gemm(dy, weight, b_mn_major=True)
        dh = _C().swiglu_bwd(da, h)
        return dh, dw, (dy if ctx.has_res else None)


def swiglu_linear_supported(h, weight) -> bool:
    return (h.is_cuda and h.dim() == 2 and h.dtype == torch.bfloat16 and h.shape[-1] % 16 == 0
            and weight.shape[0] % 8 == 0 and _ld_ok(weight) and h.is_contiguous())


def swiglu_linear(h, weight, residual=None):
    return _SwiGLULinearFn.apply(h, weight, residual)
