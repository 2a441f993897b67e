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


@pytest.mark.parametrize("m,H,n,topk", [(5, 128, 300, 64), (3, 16, 1000, 200), (4, 64, 4096, 2048), (2, 128, 77, 33)])
def test_sparse_mla_head_mean_probabilities_match_fp32(m, H, n, topk):
    """Second pass of the kernel: mean over heads of the attention probabilities of the selected slots."""
    from loongforge_b200.ops import _ext, dsa_ops

    q, kv, idx = _case(m, H, n, topk, seed=m + H + 1)
    scale = 1.0 / math.sqrt(192)
    o, pm = dsa_ops.sparse_mla_attention(q, kv, idx.long(), scale, return_head_mean_probs=True)
    _ext.check_status()
    valid = idx >= 0
    g = kv.float()[idx.clamp_min(0).long()]
    sc = torch.einsum("mhd,mkd->mhk", q.float(), g) * scale
    sc = sc.masked_fill(~valid[:, None, :], float("-inf"))
    ref = torch.nan_to_num(torch.softmax(sc, dim=-1)).mean(1)
    assert pm.shape == ref.shape and pm.dtype == torch.float32
    assert (pm - ref).abs().max().item() < 2e-3 * max(ref.max().item(), 1e-3) + 1e-6, (pm - ref).abs().max().item()
    assert pm[~valid].abs().max().item() == 0 if (~valid).any() else True
    rows = valid.any(1)
    assert (pm.sum(1)[rows] - 1).abs().max().item() < 5e-3  # a distribution over the selected slots
    ref_o, _ = _ref(q, kv, idx, scale)
    assert _rel(o, ref_o) < 2e-2


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


@pytest.mark.parametrize("m,n,Hi,topk,packed", [(300, 300, 64, 64, False), (1000, 1000, 32, 128, True),
                                                (4200, 4200, 64, 2048, False), (513, 2000, 64, 256, False)])
def test_indexer_logits_and_topk_match_fp32(m, n, Hi, topk, packed):
    """Selected sets of the native indexer (tcgen05 logits + radix select) against the fp32 formulation: the k-th
    largest logit of every row agrees and every selected key lies inside the row's causal range and scores at least
    that threshold (ties may be broken differently)."""
    from loongforge_b200.ops import _ext, dsa_ops

    torch.manual_seed(m + Hi)
    dev = "cuda"
    q = torch.randn(m, Hi, 128, device=dev).bfloat16()
    k = torch.randn(n, 128, device=dev).bfloat16()
    w = torch.randn(m, Hi, device=dev) * 0.1
    # query i sits at key position i + (n - m): it sees keys [seg start, i + n - m]
    q_pos = torch.arange(m, device=dev) + (n - m)
    k_pos = torch.arange(n, device=dev)
    seg_q = seg_k = None
    if packed:
        bounds = torch.tensor([0, 130, 131, 600, n], device=dev)
        seg_k = torch.bucketize(k_pos, bounds[1:], right=True)
        seg_q = torch.bucketize(q_pos, bounds[1:], right=True)
    idx, _ = dsa_ops.indexer_topk(q, k, w, topk, q_pos, k_pos, seg_q, seg_k, keys_in_order=True)
    _ext.check_status()
    ref_idx, ref_sc = dsa_ops.indexer_topk(q, k, w, topk, q_pos, k_pos, seg_q, seg_k, keys_in_order=False)
    logits = dsa_ops.indexer_logits_block(q, k, w)
    mask = k_pos[None, :] <= q_pos[:, None]
    if packed:
        mask &= seg_q[:, None] == seg_k[None, :]
    n_valid = mask.sum(1)
    # same number of selected keys, all of them inside the mask
    assert torch.equal((idx >= 0).sum(1), torch.minimum(n_valid, torch.tensor(topk, device=dev)))
    sel_ok = torch.gather(mask, 1, idx.clamp_min(0)) | (idx < 0)
    assert bool(sel_ok.all())
    # no duplicates
    srt = torch.sort(torch.where(idx >= 0, idx, torch.arange(-topk, 0, device=dev)[None, :].expand_as(idx)), 1).values
    assert bool((srt[:, 1:] != srt[:, :-1]).all())
    # threshold agreement: the smallest selected logit equals the reference's k-th largest (bf16 products, fp32 sums)
    got = torch.gather(logits, 1, idx.clamp_min(0)).masked_fill(idx < 0, float("inf")).min(1).values
    ref = ref_sc.masked_fill(torch.isinf(ref_sc), float("inf")).min(1).values
    rows = n_valid > 0
    assert (got[rows] - ref[rows]).abs().max().item() < 2e-2 * max(1.0, ref[rows].abs().max().item())


def test_hadamard128_kernel_matches_butterflies_and_is_its_own_inverse():
    from loongforge_b200.ops import dsa_ops

    torch.manual_seed(0)
    x = torch.randn(1000, 64, 128, device="cuda").bfloat16().requires_grad_()
    y = dsa_ops.hadamard_transform(x)
    n = 128
    h = torch.tensor([[(-1) ** bin(i & j).count("1") for j in range(n)] for i in range(n)], dtype=torch.float32, device="cuda")
    ref = x.detach().float() @ h / math.sqrt(n)
    assert _rel(y, ref) < 5e-3
    assert _rel(dsa_ops.hadamard_transform(y.detach()), x.detach()) < 1e-2  # H H = n I
    g = torch.randn_like(y)
    y.backward(g)
    assert _rel(x.grad, g.float() @ h / math.sqrt(n)) < 5e-3
