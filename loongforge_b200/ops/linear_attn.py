"""Gated delta rule (linear attention of Qwen3-Next / Qwen3.5) and the depthwise causal conv in front of it.

Per head, with state ``S [dk, dv]``, decay ``a_t = exp(g_t)`` and write strength ``beta_t``::

    S   <- a_t * S
    d_t  = beta_t * (v_t - S^T k_t)
    S   <- S + k_t d_t^T
    o_t  = S^T q_t

``gated_delta_rule_recurrent`` is that recurrence literally (the oracle); ``gated_delta_rule`` is the
chunk-parallel form (WY representation inside a chunk, one state update per chunk) that turns the
work into GEMMs. The reference calls the ``fla`` Triton kernels for this
(loongforge/models/foundation/qwen3_next/gated_deltanet.py:49-52,354); here the chunked form runs as
batched matmuls, i.e. on the tensor cores through the framework GEMM path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def gated_delta_rule_recurrent(q, k, v, g, beta, *, scale: Optional[float] = None, qk_l2norm: bool = True):
    """q, k [T, H, dk]; v [T, H, dv]; g, beta [T, H]. Returns o [T, H, dv] (fp32 math)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    q = q * (scale if scale is not None else dk ** -0.5)
    S = q.new_zeros(H, dk, dv)
    out = []
    for t in range(T):
        S = S * g[t].exp()[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        d = (v[t] - mem) * beta[t][:, None]
        S = S + k[t][:, :, None] * d[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out, 0)


def _chunk_one(q, k, v, g, beta, chunk: int):
    """One sequence, tensors already head-major: q, k [H, T, dk]; v [H, T, dv]; g, beta [H, T]."""
    H, T, dk = q.shape
    dv = v.shape[-1]
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    n = (T + pad) // chunk
    q, k, v = (t.reshape(H, n, chunk, -1) for t in (q, k, v))
    g, beta = g.reshape(H, n, chunk), beta.reshape(H, n, chunk)
    gc = g.cumsum(-1)
    k_beta, v_beta = k * beta[..., None], v * beta[..., None]
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
    decay = (gc[..., :, None] - gc[..., None, :]).masked_fill(~tri, float("-inf")).exp()
    L = (k_beta @ k.transpose(-1, -2) * decay).masked_fill(~strict, 0.0)
    eye = torch.eye(chunk, dtype=L.dtype, device=L.device)
    # WY representation of the chunk: (I + L)^-1, unit lower triangular
    A = torch.linalg.solve_triangular(L + eye, eye.expand_as(L), upper=False, unitriangular=True)
    value = A @ v_beta
    k_cum = A @ (k_beta * gc.exp()[..., None])
    S = q.new_zeros(H, dk, dv)
    outs = []
    for c in range(n):
        qc, kc, gcc = q[:, c], k[:, c], gc[:, c]
        local = (qc @ kc.transpose(-1, -2) * decay[:, c]).masked_fill(~tri, 0.0)
        v_new = value[:, c] - k_cum[:, c] @ S
        inter = (qc * gcc.exp()[..., None]) @ S
        outs.append(inter + local @ v_new)
        last = gcc[:, -1]
        S = S * last.exp()[:, None, None] + (kc * (last[:, None] - gcc).exp()[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, 1).reshape(H, n * chunk, dv)
    return o[:, :T]


def gated_delta_rule(q, k, v, g, beta, *, cu_seqlens=None, scale: Optional[float] = None, qk_l2norm: bool = True,
                     chunk: int = 64):
    """Chunk-parallel gated delta rule over packed tokens. Shapes as in the recurrent form; the state is
    reset at every boundary of ``cu_seqlens`` (host list or tensor)."""
    T, H, dk = q.shape
    dt = v.dtype
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    q = q * (scale if scale is not None else dk ** -0.5)
    bounds = [0, T] if cu_seqlens is None else [int(b) for b in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens)
                                                                  else cu_seqlens)]
    outs = []
    for s, e in zip(bounds, bounds[1:]):
        if e > s:
            outs.append(_chunk_one(q[s:e].transpose(0, 1), k[s:e].transpose(0, 1), v[s:e].transpose(0, 1),
                                   g[s:e].t(), beta[s:e].t(), chunk).transpose(0, 1))
    return torch.cat(outs, 0).to(dt)


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, cu_seqlens=None,
                  activation: Optional[str] = "silu") -> torch.Tensor:
    """Depthwise causal convolution over packed tokens. x [T, C]; weight [C, K]. Token t sees t-K+1..t of
    its own sequence only."""
    T, C = x.shape
    K = weight.shape[-1]
    bounds = [0, T] if cu_seqlens is None else [int(b) for b in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens)
                                                                  else cu_seqlens)]
    outs = []
    for s, e in zip(bounds, bounds[1:]):
        if e > s:
            seg = F.pad(x[s:e].t().unsqueeze(0), (K - 1, 0))
            outs.append(F.conv1d(seg, weight.unsqueeze(1).to(x.dtype), None if bias is None else bias.to(x.dtype),
                                 groups=C)[0].t())
    y = torch.cat(outs, 0)
    return F.silu(y) if activation in ("silu", "swish") else y
