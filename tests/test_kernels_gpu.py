"""Numerics of the sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
    from loongforge_b200.ops import _ext

    return _ext


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (384, 136, 200), (128, 128, 64), (1000, 776, 520)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(0)
    dev = "cuda"
    A = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    B = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    D = OF.gemm(A, B, a_mn_major=a_mn, b_mn_major=b_mn)
    _ext().check_status()
    Af = A.float().t() if a_mn else A.float()
    Bf = B.float() if b_mn else B.float().t()
    ref = Af @ Bf
    assert D.shape == (M, N)
    assert _rel_err(D, ref) < 1e-2, f"rel err {_rel_err(D, ref)}"


def test_gemm_big_and_epilogues():
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(1)
    dev = "cuda"
    M, N, K = 2048, 1536, 4096
    A = torch.randn(M, K, device=dev).bfloat16()
    B = torch.randn(N, K, device=dev).bfloat16() * 0.05
    bias = torch.randn(N, device=dev).bfloat16()
    res = torch.randn(M, N, device=dev).bfloat16()
    ref = A.float() @ B.float().t()
    D = OF.gemm(A, B, bias=bias, residual=res)
    assert _rel_err(D, ref + bias.float() + res.float()) < 1e-2
    acc = torch.ones(M, N, device=dev, dtype=torch.float32)
    OF.gemm(A, B, out=acc, out_mode=2)
    assert _rel_err(acc, ref + 1.0) < 2e-3
    D32 = OF.gemm(A, B, out_mode=1, alpha=0.5)
    assert _rel_err(D32, 0.5 * ref) < 2e-3
    _ext().check_status()


def test_linear_autograd_matches_torch():
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(2)
    dev = "cuda"
    x = torch.randn(512, 1024, device=dev).bfloat16().requires_grad_()
    w = (torch.randn(768, 1024, device=dev) * 0.05).bfloat16().requires_grad_()
    y = OF.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("T,H", [(64, 4096), (300, 1280), (17, 8192), (128, 128), (5000, 64), (9001, 128), (777, 256)])
def test_rmsnorm(T, H):
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(3)
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    y = OF.rmsnorm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_packed(interleaved):
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(4)
    T, g, r, d = 96, 2, 4, 128
    x = torch.randn(T, g * (r + 2) * d, device="cuda").bfloat16()
    freqs = OF.rope_freqs(torch.arange(T, device="cuda"), d, 10000.0)
    xa = x.clone().requires_grad_()
    y = OF.rope(xa * 1.0, freqs, group=r + 2, rope_in_group=r + 1, interleaved=interleaved, head_dim=d, inplace=True)
    grad = torch.randn_like(y)
    y.backward(grad)
    xc = x.cpu().float().requires_grad_()
    yr = OF.rope(xc, freqs.cpu(), group=r + 2, rope_in_group=r + 1, interleaved=interleaved, head_dim=d)
    yr.backward(grad.cpu().float())
    assert _rel_err(y.cpu(), yr) < 1e-2
    assert _rel_err(xa.grad.cpu(), xc.grad) < 1e-2


def test_swiglu():
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(5)
    x = torch.randn(200, 2 * 1376, device="cuda").bfloat16().requires_grad_()
    y = OF.swiglu(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    a, b = xr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2


def test_linear_cross_entropy():
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(6)
    T, H, V = 700, 512, 4096
    h = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.05).bfloat16().requires_grad_()
    labels = torch.randint(0, V - 100, (T,), device="cuda")
    mask = (torch.rand(T, device="cuda") > 0.2).float()
    losses = OF.linear_cross_entropy(h, w, labels, mask, valid_vocab=V - 100, chunk_tokens=256)
    c = 1.0 / mask.sum()
    (losses * mask).sum().mul(c).backward()
    hr = h.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    logits = (hr @ wr.t())[:, : V - 100]
    lr = torch.nn.functional.cross_entropy(logits, labels, reduction="none")
    (lr * mask).sum().mul(c).backward()
    assert _rel_err(losses, lr) < 2e-2
    assert _rel_err(h.grad, hr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("gdt,mdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_adam(gdt, mdt):
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(7)
    n = 100_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(gdt)
    m = torch.zeros(n, device="cuda", dtype=mdt)
    v = torch.zeros(n, device="cuda", dtype=mdt)
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr, mr, vr = p.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    for step in (1, 2):
        OF.adam_step(p, g, m, v, out, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                     grad_scale=0.5)
        OF.adam_step(pr, g.cpu(), mr, vr, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                     step=step, grad_scale=0.5)
    assert _rel_err(p.cpu(), pr) < (1e-5 if mdt == torch.float32 else 1e-3)
    assert _rel_err(out.cpu(), pr) < 1e-2
    ss = OF.sum_of_squares(g)
    assert abs(ss.item() - g.float().pow(2).sum().item()) / ss.item() < 1e-3


def _attn_ref(q, k, v, causal, scale, cu):
    from loongforge_b200.ops import functional as OF

    return OF.attention_ref(q.float(), k.float(), v.float(), causal, scale, cu)


@pytest.mark.parametrize("T,Hq,Hkv,causal", [(256, 4, 2, True), (384, 2, 2, False), (200, 8, 2, True),
                                             (1024, 4, 1, True)])
def test_attention_fwd_bwd(T, Hq, Hkv, causal):
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(10)
    dev = "cuda"
    q = torch.randn(T, Hq, 128, device=dev).bfloat16().requires_grad_()
    k = torch.randn(T, Hkv, 128, device=dev).bfloat16().requires_grad_()
    v = torch.randn(T, Hkv, 128, device=dev).bfloat16().requires_grad_()
    OF.set_attention_impl("native")
    try:
        o = OF.attention(q, k, v, causal=causal)
        do = torch.randn_like(o)
        o.backward(do)
    finally:
        OF.set_attention_impl("auto")
    _ext().check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _attn_ref(qr, kr, vr, causal, 1.0 / math.sqrt(128), None)
    ref.backward(do.float())
    assert _rel_err(o, ref) < 2e-2, f"o {_rel_err(o, ref)}"
    assert _rel_err(q.grad, qr.grad) < 3e-2, f"dq {_rel_err(q.grad, qr.grad)}"
    assert _rel_err(k.grad, kr.grad) < 3e-2, f"dk {_rel_err(k.grad, kr.grad)}"
    assert _rel_err(v.grad, vr.grad) < 3e-2, f"dv {_rel_err(v.grad, vr.grad)}"


def test_attention_packed_varlen():
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(11)
    dev = "cuda"
    G, R = 2, 3
    lens = [130, 256, 77, 300]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    qkv = torch.randn(T, G * (R + 2) * 128, device=dev).bfloat16().requires_grad_()
    o = OF.attention_packed(qkv, G, R, causal=True, cu_seqlens=cu)
    do = torch.randn_like(o)
    o.backward(do)
    _ext().check_status()
    x = qkv.detach().float().requires_grad_()
    pk = x.view(T, G, R + 2, 128)
    ref = _attn_ref(pk[:, :, :R].reshape(T, G * R, 128), pk[:, :, R], pk[:, :, R + 1], True, 1.0 / math.sqrt(128), cu)
    ref.backward(do.float())
    assert _rel_err(o, ref) < 2e-2, f"o {_rel_err(o, ref)}"
    assert _rel_err(qkv.grad, x.grad) < 3e-2, f"dqkv {_rel_err(qkv.grad, x.grad)}"


def test_gpt_model_gpu_matches_cpu():
    """Whole tiny model: loss and gradients of the native-kernel path against the CPU reference path."""
    from loongforge_b200.models.gpt import GPTModel
    from loongforge_b200.models.config import TransformerConfig

    cfg = TransformerConfig(num_layers=2, hidden_size=512, num_attention_heads=4, num_query_groups=2,
                            kv_channels=128, ffn_hidden_size=1024, vocab_size=2048, rotary_base=10000.0,
                            params_dtype=torch.bfloat16)
    torch.manual_seed(0)
    m_cpu = GPTModel(cfg)
    m_gpu = GPTModel(cfg, device="cuda")
    m_gpu.load_state_dict(m_cpu.state_dict())
    T = 384
    tokens = torch.randint(0, 2048, (T,))
    labels = torch.randint(0, 2048, (T,))
    pos = torch.arange(T)
    mask = torch.ones(T)
    lc = m_cpu(tokens, pos, labels=labels, loss_mask=mask).mean()
    lc.backward()
    lg = m_gpu(tokens.cuda(), pos.cuda(), labels=labels.cuda(), loss_mask=mask.cuda()).mean()
    lg.backward()
    _ext().check_status()
    assert abs(lc.item() - lg.item()) < 5e-2, (lc.item(), lg.item())
    for (n, pc), (_, pg) in zip(m_cpu.named_parameters(), m_gpu.named_parameters()):
        e = _rel_err(pg.grad.cpu(), pc.grad)
        assert e < 0.15, f"{n}: {e}"


@pytest.mark.parametrize("tpe", [[300, 0, 129, 1, 64, 530], [128, 128], [0, 0, 77]])
@pytest.mark.parametrize("fused_main_grad", [False, True])
def test_grouped_gemm_experts(tpe, fused_main_grad):
    """One-launch grouped GEMM (forward, dgrad, wgrad) against a per-expert fp32 loop; ragged and empty experts."""
    from loongforge_b200.ops import moe_ops

    torch.manual_seed(0)
    K, N = 264, 520
    T = sum(tpe)
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_(True)
    ws = [torch.nn.Parameter((torch.randn(N, K, device="cuda") * 0.05).bfloat16()) for _ in tpe]
    if fused_main_grad:
        for w in ws:
            w.main_grad = torch.full((N, K), 0.5, device="cuda", dtype=torch.float32)
    y = moe_ops.grouped_linear(x, ws, tpe)
    dy = torch.randn_like(y)
    y.backward(dy)
    _ext().check_status()
    s = 0
    for e, n in enumerate(tpe):
        xe, dye = x.detach()[s:s + n].float(), dy[s:s + n].float()
        if n:
            assert _rel_err(y[s:s + n], xe @ ws[e].float().t()) < 1e-2
            assert _rel_err(x.grad[s:s + n], dye @ ws[e].float()) < 1e-2
        ref_w = dye.t() @ xe
        if fused_main_grad:
            assert ws[e].grad is None
            assert torch.allclose(ws[e].main_grad, ref_w + 0.5, rtol=2e-2, atol=2e-2), e
        else:
            assert torch.allclose(ws[e].grad.float(), ref_w, rtol=3e-2, atol=6e-2), e
        s += n


@pytest.mark.parametrize("score,pre,groups,bias", [("softmax", False, None, False), ("softmax", True, None, True),
                                                   ("sigmoid", False, (8, 4), True), ("sigmoid", False, None, False),
                                                   ("softmax", False, (4, 2), False)])
@pytest.mark.parametrize("E,k", [(128, 8), (256, 8), (64, 6)])
def test_router_kernel(score, pre, groups, bias, E, k):
    """Router kernel (scores, group-limited top-k, dense outputs, backward) against the PyTorch routing math."""
    from loongforge_b200.ops import moe_ops

    torch.manual_seed(1)
    T = 333
    logits = (torch.randn(T, E, device="cuda") * 2).requires_grad_(True)
    eb = torch.randn(E, device="cuda") * 0.1 if bias else None
    ng, gk = groups if groups else (None, None)
    kw = dict(score_function=score, pre_softmax=pre, expert_bias=eb, num_groups=ng, group_topk=gk, scaling_factor=2.5)
    probs, rmap, aux = moe_ops.topk_routing(logits, k, **kw)
    w1, w2 = torch.randn_like(probs), torch.randn_like(aux)
    ((probs * w1).sum() + (aux * w2).sum()).backward()
    g_native = logits.grad.clone()
    lc = logits.detach().cpu().requires_grad_(True)
    pr, mr, ar = moe_ops.topk_routing(lc, k, **{**kw, "expert_bias": None if eb is None else eb.cpu()})
    ((pr * w1.cpu()).sum() + (ar * w2.cpu()).sum()).backward()
    assert torch.equal(rmap.cpu(), mr)
    assert torch.allclose(probs.cpu(), pr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(aux.cpu(), ar, rtol=1e-4, atol=1e-6)
    assert torch.allclose(g_native.cpu(), lc.grad, rtol=1e-3, atol=1e-4), (g_native.cpu() - lc.grad).abs().max()
