"""DeepSeek sparse attention (DSA) math: lightning indexer, top-k selection, top-k sparse MLA
attention on the absorbed (compressed-KV) form, and the indexer KL loss.

The formulas are those of the reference's torch oracles: indexer logits
``sum_h w[m,h] * relu(q[m,h,:] . k[n,:])`` (ops/tilelang_ops/lightning_indexer.py:12-32), sparse
attention over gathered KV rows with ``d_v = 512`` of the 576-dim key
(ops/tilelang_ops/sparse_mla_fwd.py:218-265), and the KL between the head-averaged attention
distribution over the selected tokens and the softmax of the index scores
(loongforge/models/common/experimental_attention_variant/dsa_fused.py:924-956). Query rows are
processed in blocks so that no ``[s_q, s_k]`` matrix larger than a block is ever alive.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


class _Hadamard128Fn(torch.autograd.Function):
    """H_128 / sqrt(128) is symmetric and orthogonal: the backward is the same kernel on the gradient."""

    @staticmethod
    def forward(ctx, x):
        from . import _ext
        return _ext.require().hadamard128(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        from . import _ext
        return _ext.require().hadamard128(g.contiguous())


def hadamard_transform(x: torch.Tensor) -> torch.Tensor:
    """x @ H_n / sqrt(n) on the last dim (n a power of two), fast Walsh-Hadamard butterflies; rows of 128 bf16 on a
    GPU run on the warp-shuffle kernel (csrc/elementwise.cu), as the indexer's rotation does."""
    n = x.shape[-1]
    assert n & (n - 1) == 0
    if n == 128 and x.is_cuda and x.dtype == torch.bfloat16:
        from . import _ext
        mod = _ext.get()
        if mod is not None and hasattr(mod, "hadamard128"):
            return _Hadamard128Fn.apply(x)
    y = x.float().reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        a, b = y[:, :, 0, :], y[:, :, 1, :]
        y = torch.stack([a + b, a - b], dim=2).reshape(-1, n)
        h *= 2
    return (y / math.sqrt(n)).reshape(x.shape).to(x.dtype)


def quant_fp8_rowwise_pow2(x: torch.Tensor, block: int = 128, eps: float = 1e-12):
    """1 x `block` e4m3 quantisation with power-of-two scales (emulated; returns dequantised values
    and scales), as the indexer inputs are quantised in the reference (dsa_fused_kernels.py:2308-2315)."""
    shp = x.shape
    xb = x.float().reshape(-1, shp[-1] // block, block)
    amax = xb.abs().amax(-1, keepdim=True).clamp_min(eps)
    scale = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    q = (xb / scale).to(torch.float8_e4m3fn).float()
    return (q * scale).reshape(shp), scale.reshape(*shp[:-1], shp[-1] // block)


def indexer_logits_block(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """q [m, Hi, D], k [n, D], w [m, Hi] -> logits [m, n] = sum_h w * relu(q . k)."""
    s = torch.einsum("mhd,nd->mhn", q.float(), k.float())
    return (torch.relu(s) * w.float().unsqueeze(-1)).sum(1)


_TK_MAX_ROW = 49152  # longest key range the selection kernel holds in shared memory


def _native_indexer(q, k) -> bool:
    from . import _ext
    mod = _ext.get()
    return (mod is not None and hasattr(mod, "indexer_topk") and q.is_cuda and q.dtype == torch.bfloat16
            and k.dtype == torch.bfloat16 and q.shape[-1] == 128 and q.shape[1] in (32, 64, 128, 256))


def indexer_topk_native(q, k, w, topk: int, k_start: torch.Tensor, k_end: torch.Tensor, max_len: int,
                        chunk: int = 4096) -> torch.Tensor:
    """Top-k key indices (int32 [m, topk], unordered, -1 padded) of every query over its key range [k_start, k_end):
    the tcgen05 logits kernel fills a [chunk, n] fp32 buffer for `chunk` queries at a time (never [m, n]) and the
    radix-select kernel picks from each row's range (csrc/dsa_sm100.cu)."""
    from . import _ext
    C = _ext.require()
    m, n = q.shape[0], k.shape[0]
    ld = (n + 3) // 4 * 4
    logits = torch.empty(min(chunk, m), ld, dtype=torch.float32, device=q.device)
    out = torch.empty(m, topk, dtype=torch.int32, device=q.device)
    st = _ext.status_tensor(q.device)
    qc, kc, wc = q.contiguous(), k.contiguous(), w.float().contiguous()
    ks, ke = k_start.to(torch.int32).contiguous(), k_end.to(torch.int32).contiguous()
    for s in range(0, m, chunk):
        e = min(m, s + chunk)
        C.indexer_topk(qc[s:e], kc, wc[s:e], ks[s:e], ke[s:e], logits, out[s:e], int(max_len), st)
    return out


def indexer_topk(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, topk: int, q_pos: torch.Tensor,
                 k_pos: torch.Tensor, seg_q: Optional[torch.Tensor] = None, seg_k: Optional[torch.Tensor] = None,
                 block: int = 1024, keys_in_order: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Causal top-k key indices per query. Returns (indices [m, topk] int64 with -1 padding,
    scores [m, topk] fp32 with -inf padding). `q_pos` / `k_pos` are global positions; `seg_*`
    optional packed-sequence ids. With ``keys_in_order`` (keys sorted by position, sequences contiguous) every
    query's candidates are one index range and a GPU runs the native kernels; the scores are then not returned
    (None): callers that need them evaluate `indexer_scores_at` on the selection."""
    m, n = q.shape[0], k.shape[0]
    if keys_in_order and n <= _TK_MAX_ROW and _native_indexer(q, k):
        kp = k_pos.contiguous()
        k_end = torch.searchsorted(kp, q_pos.contiguous(), right=True)
        if seg_q is not None:
            # keys of one sequence are contiguous: the range starts at the sequence's first key
            k_start = torch.searchsorted(seg_k.contiguous(), seg_q.contiguous(), right=False)
        else:
            k_start = torch.zeros_like(k_end)
        return indexer_topk_native(q, k, w, topk, k_start, k_end, n).long(), None
    kk = min(topk, n)
    idx_out = torch.full((m, topk), -1, dtype=torch.int64, device=q.device)
    sc_out = torch.full((m, topk), float("-inf"), dtype=torch.float32, device=q.device)
    for s in range(0, m, block):
        e = min(m, s + block)
        lg = indexer_logits_block(q[s:e], k, w[s:e])
        mask = k_pos[None, :] <= q_pos[s:e, None]
        if seg_q is not None:
            mask &= seg_q[s:e, None] == seg_k[None, :]
        lg = lg.masked_fill(~mask, float("-inf"))
        v, i = lg.topk(kk, dim=-1)
        i = torch.where(torch.isinf(v), torch.full_like(i, -1), i)
        idx_out[s:e, :kk] = i
        sc_out[s:e, :kk] = v
    return idx_out, sc_out


def _sparse_mla_block(q, idx, kv, scale: float, d_v: int, with_probs: bool):
    """One query block: returns o flattened to [b, H*d_v], with the head-mean probabilities [b, K] appended."""
    valid = idx >= 0
    g = kv[idx.clamp_min(0)]  # [b, K, Dk]
    sc = torch.einsum("bhd,bkd->bhk", q.float(), g.float()) * scale
    sc = sc.masked_fill(~valid[:, None, :], float("-inf"))
    p = torch.nan_to_num(torch.softmax(sc, dim=-1))
    o = torch.einsum("bhk,bkd->bhd", p, g[..., :d_v].float()).to(q.dtype).flatten(1)
    return torch.cat([o, p.mean(1).to(o.dtype)], dim=-1) if with_probs else o


def _native_sparse_mla(q, kv, d_v) -> bool:
    from . import _ext
    mod = _ext.get()
    return (mod is not None and hasattr(mod, "sparse_mla_fwd") and q.is_cuda and q.dtype == torch.bfloat16
            and kv.dtype == torch.bfloat16 and q.shape[-1] == 576 and d_v == 512 and q.shape[1] <= 128)


def _bmm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched product of bf16 operands on the tensor cores with an fp32 result (plain fp32 product elsewhere)."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        try:
            return torch.bmm(a, b, out_dtype=torch.float32)
        except (TypeError, NotImplementedError, RuntimeError):  # a PyTorch without the out_dtype overload
            pass
    return torch.bmm(a.float(), b.float())


def sparse_mla_backward_block(q, kv, idx, o, lse, do, scale: float, dkv: torch.Tensor, d_v: int = 512):
    """Backward of one query block given the forward's output and log-sum-exp: five batched GEMMs over the gathered
    rows, no autograd graph. q [b, H, Dk], idx [b, K] (-1 = empty), o / do [b, H, d_v], lse [b, H] (natural log);
    returns dq and ADDS the block's key / value gradient into `dkv` [n, Dk] fp32 (``index_add_``: on a GPU the order of
    the additions, hence the last bits, can differ between runs)."""
    valid = idx >= 0
    gi = idx.clamp_min(0)
    g = kv[gi]                                                      # [b, K, Dk]
    s = _bmm_f32(q, g.transpose(1, 2)) * scale                      # [b, H, K] fp32
    fin = torch.isfinite(lse)
    p = torch.exp(s - torch.where(fin, lse, torch.zeros_like(lse)).unsqueeze(-1))
    p = p * (valid.unsqueeze(1) & fin.unsqueeze(-1))
    dp = _bmm_f32(do, g[..., :d_v].transpose(1, 2))                 # [b, H, K]
    delta = (do.float() * o.float()).sum(-1, keepdim=True)          # [b, H, 1]
    ds = (p * (dp - delta) * scale).to(q.dtype)
    pb = p.to(q.dtype)
    dq = _bmm_f32(ds, g)                                            # [b, H, Dk]
    dg = _bmm_f32(ds.transpose(1, 2), q)                            # [b, K, Dk]
    dg[..., :d_v] += _bmm_f32(pb.transpose(1, 2), do)
    dkv.index_add_(0, gi.reshape(-1), dg.reshape(-1, dg.shape[-1]))  # empty slots carry p = ds = 0
    return dq.to(q.dtype)


class _SparseMlaFn(torch.autograd.Function):
    """Forward on the tcgen05 kernel (csrc/dsa_sm100.cu): no gathered [rows, K, 576] tensor ever exists. Backward works
    one query block at a time from the saved output and log-sum-exp (`sparse_mla_backward_block`: batched tensor-core
    GEMMs over the block's gathered rows), so only one block's gathered keys are alive."""

    @staticmethod
    def forward(ctx, q, kv, indices, scale, block):
        from . import _ext
        qc = q if (q.stride(2) == 1 and q.stride(1) % 8 == 0 and q.stride(0) % 8 == 0) else q.contiguous()
        kc = kv if (kv.stride(1) == 1 and kv.stride(0) % 8 == 0) else kv.contiguous()
        o, lse = _ext.require().sparse_mla_fwd(qc, kc, indices.to(torch.int32).contiguous(), float(scale),
                                               _ext.status_tensor(q.device))
        ctx.save_for_backward(q, kv, indices, o, lse)
        ctx.cfg = (scale, block)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, kv, indices, o, lse = ctx.saved_tensors
        scale, block = ctx.cfg
        dq = torch.empty_like(q)
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=kv.device)
        kvd = kv.detach()
        for s in range(0, q.shape[0], block):
            e = min(q.shape[0], s + block)
            dq[s:e] = sparse_mla_backward_block(q[s:e].detach(), kvd, indices[s:e].long(), o[s:e], lse[s:e],
                                                do[s:e].contiguous(), scale, dkv)
        return dq, dkv.to(kv.dtype), None, None, None


def sparse_mla_head_mean_probs(q, kv, indices, lse, scale: float) -> torch.Tensor:
    """Head-averaged attention probabilities of the selected slots [m, K] fp32 (a constant: no gradient), from a second
    pass of the sparse attention kernel that takes the forward's log-sum-exp as input (csrc/dsa_sm100.cu)."""
    from . import _ext
    qd, kd = q.detach(), kv.detach()
    qc = qd if (qd.stride(2) == 1 and qd.stride(1) % 8 == 0 and qd.stride(0) % 8 == 0) else qd.contiguous()
    kc = kd if (kd.stride(1) == 1 and kd.stride(0) % 8 == 0) else kd.contiguous()
    return _ext.require().sparse_mla_probs(qc, kc, indices.to(torch.int32).contiguous(), lse.detach().contiguous(),
                                           float(scale), _ext.status_tensor(q.device))


def sparse_mla_attention(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, scale: float, d_v: int = 512,
                         block: int = 256, return_head_mean_probs: bool = False):
    """q [m, H, Dk], kv [n, Dk] (shared by all heads), indices [m, K] (-1 = empty).
    Returns o [m, H, d_v] (and the head-averaged attention distribution over the K slots, a constant target).
    On a GPU the forward (and, when asked for, the head-mean distribution) run on the tcgen05 kernels; query blocks are
    recomputed in backward (``ops/blockwise.py``), so the gathered keys of only one block are alive."""
    from .blockwise import blockwise_apply

    if _native_sparse_mla(q, kv, d_v):
        o, lse = _SparseMlaFn.apply(q, kv, indices, scale, block)
        if not return_head_mean_probs:
            return o
        return o, sparse_mla_head_mean_probs(q, kv, indices, lse, scale)
    m, H, _ = q.shape
    K = indices.shape[1]
    fn = lambda qb, ib, kvv: _sparse_mla_block(qb, ib, kvv, scale, d_v, return_head_mean_probs)  # noqa: E731
    out = blockwise_apply(fn, [q, indices], [kv], block)
    o = out[:, :H * d_v].reshape(m, H, d_v)
    if return_head_mean_probs:
        return o, out[:, H * d_v:H * d_v + K].detach().float()
    return o


class _IndexerScoresFn(torch.autograd.Function):
    """Index scores at the selected slots, one query block at a time, without an autograd graph over the gathered keys:
    forward keeps only the [m, K] result; backward recomputes a block's scores and forms the three gradients with
    batched GEMMs (reference kernels: ops/tilelang_ops/lightning_indexer.py:170-347, restricted to the selection)."""

    @staticmethod
    def _block(qb, kk, ib):
        kg = kk[ib.clamp_min(0)]                                     # [b, K, D]
        return kg, _bmm_f32(qb, kg.transpose(1, 2))                  # [b, Hi, K] fp32

    @staticmethod
    def forward(ctx, qi, wi, ki, indices, block):
        out = torch.empty(indices.shape, dtype=torch.float32, device=qi.device)
        for s in range(0, qi.shape[0], block):
            e = min(qi.shape[0], s + block)
            _, sc = _IndexerScoresFn._block(qi[s:e], ki, indices[s:e])
            out[s:e] = (torch.relu(sc) * wi[s:e].float().unsqueeze(-1)).sum(1)
        ctx.save_for_backward(qi, wi, ki, indices)
        ctx.block = block
        return out

    @staticmethod
    def backward(ctx, d_out):
        qi, wi, ki, indices = ctx.saved_tensors
        dq = torch.empty_like(qi)
        dw = torch.empty(wi.shape, dtype=torch.float32, device=wi.device)
        dk = torch.zeros(ki.shape, dtype=torch.float32, device=ki.device)
        for s in range(0, qi.shape[0], ctx.block):
            e = min(qi.shape[0], s + ctx.block)
            ib = indices[s:e]
            kg, sc = _IndexerScoresFn._block(qi[s:e], ki, ib)
            g = (d_out[s:e].float() * (ib >= 0)).unsqueeze(1)        # [b, 1, K]; empty slots carry no gradient
            dw[s:e] = (torch.relu(sc) * g).sum(-1)
            ds = (g * wi[s:e].float().unsqueeze(-1) * (sc > 0)).to(qi.dtype)   # [b, Hi, K]
            dq[s:e] = _bmm_f32(ds, kg).to(qi.dtype)
            dk.index_add_(0, ib.clamp_min(0).reshape(-1), _bmm_f32(ds.transpose(1, 2), qi[s:e]).reshape(-1, ki.shape[-1]))
        return dq, dw.to(wi.dtype), dk.to(ki.dtype), None, None


def indexer_scores_at(qi: torch.Tensor, wi: torch.Tensor, ki: torch.Tensor, indices: torch.Tensor,
                      block: int = 256) -> torch.Tensor:
    """Index scores ``sum_h w * relu(q_h . k)`` at the selected slots only: [m, K] fp32, differentiable w.r.t. the
    indexer projections, evaluated (and differentiated) in query blocks so that only one block's gathered keys are
    alive."""
    return _IndexerScoresFn.apply(qi, wi, ki, indices, block)


def indexer_kl_loss(index_scores: torch.Tensor, attn_probs_head_mean: torch.Tensor, indices: torch.Tensor,
                    coeff: float) -> torch.Tensor:
    """KL( attention distribution || softmax(index scores) ) over the selected slots, summed over
    slots and queries, divided by the number of queries, times `coeff`. The attention side is a
    constant target (detached)."""
    valid = indices >= 0
    tgt = attn_probs_head_mean.detach().float()
    logq = torch.log_softmax(index_scores.float().masked_fill(~valid, float("-inf")), dim=-1)
    logq = torch.where(valid, logq, torch.zeros_like(logq))
    logp = torch.where(tgt > 0, torch.log(tgt.clamp_min(1e-30)), torch.zeros_like(tgt))
    kl = (tgt * (logp - logq) * valid).sum()
    return kl / max(index_scores.shape[0], 1) * coeff
