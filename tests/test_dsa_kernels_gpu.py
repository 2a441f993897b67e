"""DeepSeek sparse attention forward kernel (tcgen05, heads as tile rows, gathered keys) against the fp32 PyTorch
formulation of the same op: ragged top-k lists with -1 padding, head counts below the tile height, a top-k that is
not a multiple of the block, tokens that select nothing; and the gradients of the autograd wrapper."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _ref(q, kv, idx, scale):
    valid = idx >= 0
    g = kv.float()[idx.clamp_min(0).long()]                       # [m, K, 576]
    sc = torch.einsum("mhd,mkd->mhk", q.float(), g) * scale
    sc = sc.masked_fill(~valid[:, None, :], float("-inf"))
    lse = torch.logsumexp(sc, dim=-1)
    p = torch.nan_to_num(torch.softmax(sc, dim=-1))
    return torch.einsum("mhk,mkd->mhd", p, g[..., :512]), lse


def _case(m, H, n, topk, seed, ragged=True):
    torch.manual_seed(seed)
    dev = "cuda"
    q = (torch.randn(m, H, 576, device=dev) * 0.5).bfloat16()
    kv = (torch.randn(n, 576, device=dev) * 0.5).bfloat16()
    idx = torch.stack([torch.randperm(n, device=dev)[:topk] for _ in range(m)]).int()
    if ragged:
        keep = torch.randint(0, topk + 1, (m,), device=dev)
        keep[0] = 0  # a token that selects nothing
        idx = torch.where(torch.arange(topk, device=dev)[None, :] < keep[:, None], idx, torch.full_like(idx, -1))
    return q, kv, idx


@pytest.mark.parametrize("m,H,n,topk", [(5, 128, 300, 64), (3, 16, 1000, 200), (4, 64, 4096, 2048), (2, 128, 77, 33)])
def test_sparse_mla_forward_matches_fp32(m, H, n, topk):
    from loongforge_b200.ops import _ext

    q, kv, idx = _case(m, H, n, topk, seed=m + H)
    scale = 1.0 / math.sqrt(192)
    o, lse = _ext.require().sparse_mla_fwd(q, kv, idx, scale, _ext.status_tensor(q.device))
    _ext.check_status()
    ref, lse_ref = _ref(q, kv, idx, scale)
    assert _rel(o, ref) < 2e-2, _rel(o, ref)
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse), fin)
    assert (lse[fin] - lse_ref[fin]).abs().max().item() < 2e-2
    assert o[0].abs().max().item() == 0  # nothing selected -> zero output


def test_sparse_mla_autograd_wrapper():
    from loongforge_b200.ops import _ext, dsa_ops

    q, kv, idx = _case(40, 32, 500, 96, seed=3)
    scale = 1.0 / math.sqrt(192)
    qg, kg = q.clone().requires_grad_(), kv.clone().requires_grad_()
    o = dsa_ops.sparse_mla_attention(qg, kg, idx.long(), scale, block=16)
    do = torch.randn_like(o)
    o.backward(do)
    _ext.check_status()
    qr, kr = q.float().requires_grad_(), kv.float().requires_grad_()
    ref, _ = _ref(qr, kr, idx, scale)
    ref.backward(do.float())
    assert _rel(o, ref) < 2e-2
    assert _rel(qg.grad, qr.grad) < 3e-2
    assert _rel(kg.grad, kr.grad) < 3e-2
