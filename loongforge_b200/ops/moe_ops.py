"""Router and expert math of the MoE layer (PyTorch reference path + native kernels on CUDA).

Routing semantics are those of Megatron's ``topk_softmax_with_capacity`` as copied in the
reference (loongforge/models/foundation/ernie4_5_vl/ernie_router.py:32-140): softmax routing either
before the top-k over all experts or after it over the selected k; sigmoid routing with scores
normalised over the selected k; an optional selection-only expert bias; group-limited top-k;
a final scaling factor. Outputs are dense ``probs [T, E]`` (zero off the top-k) and a boolean
``routing_map [T, E]``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import functional as OF


def group_limited_topk(scores: torch.Tensor, topk: int, num_groups: int, group_topk: int):
    T, E = scores.shape
    per = E // num_groups
    group_scores = scores.view(T, num_groups, per).topk(max(topk // group_topk, 1), dim=-1).values.sum(-1)
    gidx = group_scores.topk(group_topk, dim=-1).indices
    gmask = torch.zeros_like(group_scores).scatter_(1, gidx, 1.0)
    mask = gmask.unsqueeze(-1).expand(T, num_groups, per).reshape(T, E).bool()
    masked = scores.masked_fill(~mask, float("-inf"))
    return masked.topk(topk, dim=-1)


_SCORE_CODE = {("softmax", False): 0, ("softmax", True): 1, ("sigmoid", False): 2, ("sigmoid", True): 2}


class _RouterFn(torch.autograd.Function):
    """Score + (group-limited) top-k + dense outputs in one launch (csrc/router.cu)."""

    @staticmethod
    def forward(ctx, logits, bias, topk, code, num_groups, group_topk, scale):
        from . import _ext

        logits = logits.contiguous()
        probs, rmap, aux, idx, counts = _ext.require().router_fwd(logits, bias, topk, code, num_groups, group_topk, scale)
        ctx.save_for_backward(logits, rmap)
        ctx.cfg = (topk, code, scale)
        ctx.mark_non_differentiable(rmap, idx, counts)
        return probs, rmap, aux, idx, counts

    @staticmethod
    def backward(ctx, dprobs, _dmap, daux, _didx, _dcounts):
        from . import _ext

        logits, rmap = ctx.saved_tensors
        topk, code, scale = ctx.cfg
        dl = _ext.require().router_bwd(logits, rmap, dprobs.float().contiguous(),
                                       None if daux is None else daux.float().contiguous(), topk, code, scale)
        return dl.to(logits.dtype), None, None, None, None, None, None


def _router_native_ok(logits, topk, num_groups) -> bool:
    return (logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and logits.shape[1] <= 512
            and topk <= 32 and (not num_groups or (num_groups <= 32 and logits.shape[1] % num_groups == 0)))


def topk_routing(logits: torch.Tensor, topk: int, *, score_function: str = "softmax", pre_softmax: bool = False,
                 expert_bias: Optional[torch.Tensor] = None, num_groups: Optional[int] = None,
                 group_topk: Optional[int] = None, scaling_factor: Optional[float] = None):
    """Returns (probs [T, E], routing_map [T, E] bool, scores used by the aux loss [T, E])."""
    if score_function not in ("softmax", "sigmoid", "sqrtsoftplus"):
        raise ValueError(f"unknown router score function {score_function}")
    if score_function != "sqrtsoftplus" and _router_native_ok(logits, topk, num_groups):
        bias = None if expert_bias is None else expert_bias.detach().float().contiguous()
        probs, rmap, aux, _, _ = _RouterFn.apply(logits, bias, topk, _SCORE_CODE[(score_function, bool(pre_softmax))],
                                                 int(num_groups or 0), int(group_topk or 0),
                                                 float(scaling_factor) if scaling_factor else 1.0)
        return probs, rmap, aux
    T, E = logits.shape

    def select(s):
        if num_groups and group_topk:
            return group_limited_topk(s, topk, num_groups, group_topk)
        return s.topk(topk, dim=-1)

    if score_function == "softmax":
        full = torch.softmax(logits, dim=-1, dtype=torch.float32)
        if pre_softmax:
            sel = full + expert_bias if expert_bias is not None else full
            _, idx = select(sel)
            vals = full.gather(1, idx)
        else:
            sel = logits + expert_bias if expert_bias is not None else logits
            v, idx = select(sel)
            vals = torch.softmax(logits.gather(1, idx), dim=-1, dtype=torch.float32)
        aux_scores = full
    elif score_function in ("sigmoid", "sqrtsoftplus"):
        # sqrtsoftplus (DeepSeek-V4): s = sqrt(softplus(logit)); selection, normalisation and aux scores as for sigmoid
        s = torch.sigmoid(logits.float()) if score_function == "sigmoid" else \
            torch.sqrt(torch.nn.functional.softplus(logits.float()))
        sel = s + expert_bias if expert_bias is not None else s
        _, idx = select(sel)
        vals = s.gather(1, idx)
        if topk > 1:
            vals = vals / (vals.sum(-1, keepdim=True) + 1e-20)
        aux_scores = s / (s.sum(-1, keepdim=True) + 1e-20)
    else:
        raise ValueError(f"unknown router score function {score_function}")
    if scaling_factor:
        vals = vals * scaling_factor
    probs = torch.zeros(T, E, dtype=torch.float32, device=logits.device).scatter(1, idx, vals)
    routing_map = torch.zeros(T, E, dtype=torch.bool, device=logits.device).scatter(1, idx, True)
    return probs, routing_map, aux_scores


def hash_routing(token_ids: torch.Tensor, num_experts: int, topk: int) -> torch.Tensor:
    """Static routing of DeepSeek-V4's first MoE layers: expert j of token t is a fixed hash of its id.
    Returns [T, topk] distinct expert indices (Knuth multiplicative hash for the first, odd stride after)."""
    t = token_ids.long()
    first = (t * 2654435761 % 4294967296) % num_experts
    stride = 2 * ((t * 40503 % 65536) % max(num_experts // 2, 1)) + 1  # odd
    if num_experts & (num_experts - 1):  # not a power of two: fall back to consecutive experts (always distinct)
        stride = torch.ones_like(stride)
    j = torch.arange(topk, device=t.device)
    return (first.unsqueeze(1) + stride.unsqueeze(1) * j) % num_experts


def switch_aux_loss(scores: torch.Tensor, tokens_per_expert: torch.Tensor, topk: int, coeff: float) -> torch.Tensor:
    """Switch-transformer load-balancing loss: E * coeff / (T^2 * k) * sum_e P_e * f_e."""
    T, E = scores.shape
    agg = scores.sum(0)
    return (agg * tokens_per_expert.to(agg.dtype)).sum() * (E * coeff / (T * T * topk))


def seq_aux_loss(scores, routing_map, topk: int, seq_lens: Sequence[int], coeff: float) -> torch.Tensor:
    """The same loss computed per sequence and averaged (DeepSeek-V3 'seq_aux_loss')."""
    total = scores.new_zeros(())
    start = 0
    for n in seq_lens:
        total = total + switch_aux_loss(scores[start:start + n], routing_map[start:start + n].sum(0), topk, coeff)
        start += n
    return total / max(len(seq_lens), 1)


def _native_grouped(x: torch.Tensor, weights) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and weights[0].shape[0] % 8 == 0
            and weights[0].shape[1] % 8 == 0)


class _GroupedLinearFn(torch.autograd.Function):
    """y[rows of expert e] = x[rows of e] @ W_e^T for tokens sorted by expert (variable rows per
    expert). On the GPU forward, dgrad and wgrad are ONE grouped tcgen05 launch each (per-expert TMA
    descriptors, ragged rows exact); wgrad accumulates into ``main_grad`` when present. Elsewhere the
    same math runs as one GEMM per non-empty expert."""

    @staticmethod
    def forward(ctx, x, tokens_per_expert, *weights):
        N = weights[0].shape[0]
        y = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        tpe = [int(n) for n in tokens_per_expert]
        ctx.native = _native_grouped(x, weights)
        if ctx.native:
            x = x.contiguous()
            OF.grouped_gemm(x, None, list(weights), [y], tpe, mode=0)
        else:
            s = 0
            for w, n in zip(weights, tpe):
                if n > 0:
                    OF.gemm(x[s:s + n], w, out=y[s:s + n])
                s += n
        ctx.save_for_backward(x, *weights)
        ctx.tpe = tpe
        return y

    @staticmethod
    def backward(ctx, dy):
        x, *weights = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        grads = []
        if ctx.native:
            OF.grouped_gemm(dy, None, weights, [dx], ctx.tpe, mode=1)
            fused = all(getattr(w, "main_grad", None) is not None for w in weights)
            if fused:
                OF.grouped_gemm(dy, x, [], [w.main_grad for w in weights], ctx.tpe, mode=2, out_mode=2)
                for w in weights:
                    hook = getattr(w, "grad_ready", None)
                    if hook is not None:
                        hook()
                grads = [None] * len(weights)
            else:
                grads = [torch.zeros_like(w) if n == 0 else torch.empty_like(w) for w, n in zip(weights, ctx.tpe)]
                OF.grouped_gemm(dy, x, [], grads, ctx.tpe, mode=2, out_mode=0)
            return (dx, None, *grads)
        s = 0
        for w, n in zip(weights, ctx.tpe):
            if n > 0:
                OF.gemm(dy[s:s + n], w, b_mn_major=True, out=dx[s:s + n])
                grads.append(OF._wgrad(dy[s:s + n], x[s:s + n], w))
            else:
                if getattr(w, "main_grad", None) is not None:
                    hook = getattr(w, "grad_ready", None)
                    if hook is not None:
                        hook()
                    grads.append(None)
                else:
                    grads.append(torch.zeros_like(w))
            s += n
        return (dx, None, *grads)


def grouped_linear(x: torch.Tensor, weights: List[torch.Tensor], tokens_per_expert: List[int]) -> torch.Tensor:
    if x.shape[0] == 0:
        return x.new_zeros(0, weights[0].shape[0]) + sum(w.sum() * 0 for w in weights)
    return _GroupedLinearFn.apply(x, tuple(tokens_per_expert), *weights)
