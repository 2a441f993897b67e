"""Diffusion transformers and objectives on CPU: shapes, invariances, objective identities, Ulysses equivalence."""
import pytest
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


def _dit_run(rank, world, name, dims_kw, steps=2):
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.diffusion_trainer import build_diffusion_trainer
    from loongforge_b200.runtime.trainer import TrainConfig

    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=64, train_iters=steps, lr=1e-3, clip_grad=1.0,
                     log_interval=1000, seed=3)
    tr = build_diffusion_trainer(name, tc, ParallelDims(**dims_kw))
    it = tr.build_data_iterator(None)
    # every layout draws the same noise for the same sample: one generator per global sample index
    out = []
    for _ in range(steps):
        m = tr.train_step(it)
        out.append((m["loss"], m["grad_norm"]))
    return out


@pytest.mark.parametrize("name,dims,world", [("tiny-wan", {"cp": 2}, 2), ("tiny-qwen-image", {}, 1)])
def test_diffusion_trainer_layouts(name, dims, world):
    """WAN under Ulysses sequence parallelism follows the single-process trajectory; Qwen-Image trains."""
    ref = run_distributed(_dit_run, 1, name, {})[0]
    res = run_distributed(_dit_run, world, name, dict(dims))
    assert all(l == l and g > 0 for l, g in ref)
    for (l0, g0), (l1, g1) in zip(ref, res[0]):
        assert abs(l0 - l1) < 1e-4 * abs(l0) and abs(g0 - g1) < 1e-3 * max(1, g0), (ref, res)


def test_diffusion_cli_and_resume(tmp_path):
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, "-m", "loongforge_b200.train", "--model-name", "tiny-wan", "--seq-length", "64",
            "--micro-batch-size", "1", "--global-batch-size", "2", "--lr", "1e-3", "--log-interval", "1",
            "--save", str(tmp_path / "ck"), "--load", str(tmp_path / "ck")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root)

    def run(iters):
        p = subprocess.run(base + ["--train-iters", str(iters)], cwd=root, capture_output=True, text=True, timeout=600,
                           env=env)
        assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
        return [int(i) for i in re.findall(r"iteration\s+(\d+)/", p.stdout)]

    assert run(2) == [1, 2]
    assert run(4) == [3, 4], "the second run resumes from the checkpoint of the first"


def test_wan_packed_samples_match_per_sample_forward_and_backward():
    """Three videos of different sizes packed into one token row give the same predictions and parameter gradients
    as three separate forward passes."""
    torch.manual_seed(0)
    m = D.WanModel(_wan_cfg())
    lats = [torch.randn(4, 2, 8, 8), torch.randn(4, 1, 4, 8), torch.randn(4, 3, 4, 4)]
    texts = [torch.randn(3, 32), torch.randn(5, 32), torch.randn(2, 32)]
    t = torch.tensor([100.0, 500.0, 900.0])
    ref = [m(l[None], t[i:i + 1], c[None])[0] for i, (l, c) in enumerate(zip(lats, texts))]
    sum(r.pow(2).sum() for r in ref).backward()
    g_ref = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    m.zero_grad()
    out = m.forward_packed(lats, t, texts)
    assert all(o.shape == r.shape and torch.allclose(o, r, atol=1e-4) for o, r in zip(out, ref))
    sum(o.pow(2).sum() for o in out).backward()
    for n, p in m.named_parameters():
        if n in g_ref:
            assert torch.allclose(p.grad, g_ref[n], atol=2e-3, rtol=1e-3), n


def test_diffusion_trainer_packs_variable_size_samples(tmp_path):
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.diffusion_trainer import build_diffusion_trainer
    from loongforge_b200.runtime.trainer import TrainConfig

    g = torch.Generator().manual_seed(0)
    for i, (f, h, w, lt) in enumerate([(2, 8, 8, 3), (1, 4, 8, 5), (3, 4, 4, 2), (2, 4, 4, 4)]):
        torch.save({"latents": torch.randn(4, f, h, w, generator=g), "text": torch.randn(lt, 32, generator=g)},
                   tmp_path / f"s{i}.pt")
    ps.destroy_model_parallel()
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=64, train_iters=3, lr=1e-3, log_interval=1000)
    tr = build_diffusion_trainer("tiny-wan", tc)
    it = tr.build_data_iterator(type("A", (), {"data_path": [str(tmp_path)]})())
    b = next(iter(it))
    assert isinstance(b["latents"], list) and b["latents"][0].shape != b["latents"][1].shape
    ms = [tr.train_step(it) for _ in range(3)]
    assert all(m["loss"] == m["loss"] and m["grad_norm"] > 0 for m in ms)
