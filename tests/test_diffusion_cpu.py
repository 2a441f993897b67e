"""Diffusion transformers and objectives on CPU: shapes, invariances, objective identities, Ulysses equivalence."""
import torch

from loongforge_b200.models import diffusion as D
from tests.dist_utils import run_distributed


def _wan_cfg(**kw):
    base = dict(hidden_size=48, num_heads=4, num_layers=2, ffn_hidden_size=96, in_channels=4, out_channels=4,
                text_dim=32, freq_dim=16)
    base.update(kw)
    return D.DiTConfig(**base)


def test_wan_patchify_roundtrip_and_forward_backward():
    torch.manual_seed(0)
    m = D.WanModel(_wan_cfg(image_context_dim=24))
    x = torch.randn(2, 4, 3, 8, 12)
    tok, grid = m.patchify(x)
    assert grid == (3, 4, 6) and torch.equal(m.unpatchify(tok, grid), x)
    out = m(x, torch.tensor([10.0, 500.0]), torch.randn(2, 7, 32), image_context=torch.randn(2, 5, 24))
    assert out.shape == x.shape
    out.pow(2).mean().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_rope_3d_is_relative():
    """Attention logits after RoPE depend only on coordinate differences."""
    torch.manual_seed(0)
    d = 24
    q, k = torch.randn(1, 1, 1, d), torch.randn(1, 1, 1, d)
    def logit(pq, pk):
        aq = D.rope_3d_angles_at(torch.tensor([pq]), d, 10000.0)
        ak = D.rope_3d_angles_at(torch.tensor([pk]), d, 10000.0)
        return (D.apply_rope_interleaved(q, aq) * D.apply_rope_interleaved(k, ak)).sum()
    assert torch.allclose(logit([1, 2, 3], [0, 0, 1]), logit([4, 7, 5], [3, 5, 3]), atol=1e-4)


def test_qwen_image_double_stream():
    torch.manual_seed(0)
    m = D.QwenImageModel(_wan_cfg())
    img = torch.randn(2, 6 * 4, 16)
    out = m(img, torch.tensor([0.3, 0.9]), torch.randn(2, 5, 32), (6, 4))
    assert out.shape == (2, 24, 16)
    out.sum().backward()
    # the text stream's output of the LAST block is discarded, so its post-attention parameters see no gradient
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert missing and all(n.startswith("blocks.1.txt.") for n in missing), missing


def test_flow_match_objective():
    s = D.FlowMatchScheduler(1000, shift=3.0)
    assert s.sigmas[0] == 1.0 and s.sigmas[-1] == 0.0 and (s.sigmas[:-1] >= s.sigmas[1:]).all()
    x0, n = torch.randn(4, 3, 2), torch.randn(4, 3, 2)
    ids = torch.tensor([0, 250, 700, 999])
    xt = s.add_noise(x0, n, ids)
    assert torch.allclose(xt[0], n[0]) and torch.allclose(xt[3], x0[3])
    assert float(s.loss(s.training_target(x0, n), x0, n, ids)) == 0.0
    # exact velocity: Euler steps along the straight path land on x0
    x, v = xt[1:2], s.training_target(x0, n)[1:2]
    for i in range(250, 1000):
        x = s.step(v, torch.tensor([i]), x)
    assert torch.allclose(x, x0[1:2], atol=1e-4)


def test_gaussian_diffusion_identities():
    g = D.GaussianDiffusion(100, "cosine")
    x0, eps = torch.randn(3, 5), torch.randn(3, 5)
    t = torch.tensor([0, 50, 99])
    xt = g.q_sample(x0, t, eps)
    assert torch.allclose(g.predict_x0_from_eps(xt, t, eps), x0, atol=1e-4)
    assert float(g.training_loss(lambda x, tt: eps, x0, t, noise=eps)) == 0.0


def _ulysses_rank(rank, world):
    import torch.distributed as dist

    torch.manual_seed(0)
    m = D.WanModel(_wan_cfg())
    x = torch.randn(1, 4, 2, 8, 8)
    t, ctx = torch.tensor([100.0]), torch.randn(1, 3, 32)
    ref = m(x, t, ctx)
    out = m(x, t, ctx, ulysses_group=dist.group.WORLD)
    out.pow(2).sum().backward()
    g = m.blocks[0].self_attn.q.weight.grad.clone()
    dist.all_reduce(g)  # each rank holds the gradient of its token shard
    m.zero_grad()
    m(x, t, ctx).pow(2).sum().backward()
    return float((out - ref).abs().max()), float((g - m.blocks[0].self_attn.q.weight.grad).abs().max())


def test_wan_ulysses_matches_single_rank():
    for err_out, err_grad in run_distributed(_ulysses_rank, 2):
        assert err_out < 1e-4 and err_grad < 1e-3, (err_out, err_grad)
