"""Hybrid-attention families (Qwen3-Next / Qwen3.5): gated delta rule numerics and a tiny end-to-end model."""
import torch

from loongforge_b200.ops import linear_attn as LA


def test_chunked_gated_delta_rule_matches_recurrence():
    torch.manual_seed(0)
    T, H, dk, dv = 150, 3, 16, 24
    q, k, v = torch.randn(T, H, dk), torch.randn(T, H, dk), torch.randn(T, H, dv)
    g = -torch.rand(T, H) * 0.5
    beta = torch.rand(T, H)
    ref = LA.gated_delta_rule_recurrent(q, k, v, g, beta)
    out = LA.gated_delta_rule(q, k, v, g, beta, chunk=32)
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-3), (out - ref).abs().max()


def test_gated_delta_rule_resets_state_at_sequence_boundaries():
    torch.manual_seed(1)
    T, H, dk, dv = 96, 2, 8, 8
    q, k, v = torch.randn(T, H, dk), torch.randn(T, H, dk), torch.randn(T, H, dv)
    g, beta = -torch.rand(T, H), torch.rand(T, H)
    cu = [0, 40, 96]
    out = LA.gated_delta_rule(q, k, v, g, beta, cu_seqlens=cu, chunk=16)
    for s, e in zip(cu, cu[1:]):
        ref = LA.gated_delta_rule_recurrent(q[s:e], k[s:e], v[s:e], g[s:e], beta[s:e])
        assert torch.allclose(out[s:e], ref, atol=2e-4, rtol=1e-3)


def test_gated_delta_rule_gradients_flow():
    torch.manual_seed(2)
    T, H, dk, dv = 40, 2, 8, 8
    q = torch.randn(T, H, dk, dtype=torch.float64, requires_grad=True)
    k = torch.randn(T, H, dk, dtype=torch.float64, requires_grad=True)
    v = torch.randn(T, H, dv, dtype=torch.float64, requires_grad=True)
    g = (-torch.rand(T, H, dtype=torch.float64)).requires_grad_()
    beta = torch.rand(T, H, dtype=torch.float64).requires_grad_()
    a = LA.gated_delta_rule(q, k, v, g, beta, chunk=8).double()
    b = LA.gated_delta_rule_recurrent(q, k, v, g, beta).double()
    w = torch.randn_like(a)
    ga = torch.autograd.grad((a * w).sum(), [q, k, v, g, beta])
    gb = torch.autograd.grad((b * w).sum(), [q, k, v, g, beta])
    for x, y in zip(ga, gb):
        assert torch.allclose(x, y, atol=1e-3, rtol=1e-2), (x - y).abs().max()


def test_causal_conv_is_causal_and_sequence_local():
    torch.manual_seed(3)
    x = torch.randn(20, 6)
    w = torch.randn(6, 4)
    y = LA.causal_conv1d(x, w, cu_seqlens=[0, 12, 20], activation=None)
    x2 = x.clone()
    x2[15:] += 1.0  # future tokens of the second sequence must not change earlier outputs
    y2 = LA.causal_conv1d(x2, w, cu_seqlens=[0, 12, 20], activation=None)
    assert torch.allclose(y[:15], y2[:15])
    x3 = x.clone()
    x3[:12] += 1.0  # the first sequence must not leak into the second
    y3 = LA.causal_conv1d(x3, w, cu_seqlens=[0, 12, 20], activation=None)
    assert torch.allclose(y[12:], y3[12:])
    manual = sum(w[:, j] * x[5 - 3 + j] for j in range(4))
    assert torch.allclose(y[5], manual, atol=1e-5)


def test_tiny_qwen3_next_trains():
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-qwen3-next")
    assert [cfg.layer_type(i) for i in range(4)] == ["linear_attention"] * 3 + ["full_attention"]
    torch.manual_seed(0)
    model = build_model(cfg)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    T = 64
    tokens = torch.randint(0, cfg.vocab_size, (T,))
    labels = torch.roll(tokens, -1)
    pos = torch.arange(T)
    losses = []
    for _ in range(8):
        loss = model(tokens, pos, labels=labels, loss_mask=torch.ones(T)).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert all(p.grad is not None for p in model.parameters())
    assert losses[-1] < losses[0] - 0.3, losses


def _train_tiny(name, steps=6):
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config(name)
    torch.manual_seed(0)
    model = build_model(cfg)
    model.train()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    T = 48
    tokens = torch.randint(0, cfg.vocab_size, (T,))
    labels, pos = torch.roll(tokens, -1), torch.arange(T)
    losses = []
    for _ in range(steps):
        loss = model(tokens, pos, labels=labels, loss_mask=torch.ones(T)).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return model, losses


def test_tiny_minimax_full_width_qk_norm_trains():
    model, losses = _train_tiny("tiny-minimax")
    att = model.decoder.layers[0].self_attention
    assert att.q_layernorm.weight.numel() == 4 * 16 and att.k_layernorm.weight.numel() == 2 * 16
    assert losses[-1] < losses[0]


def test_tiny_mimo_mtp_hidden_first_trains():
    model, losses = _train_tiny("tiny-mimo")
    assert model.mtp is not None and model.cfg.mtp_hidden_first
    assert losses[-1] < losses[0]


def test_ernie_3d_rotary_layout():
    from loongforge_b200.models.ernie import ernie_3d_angles

    pos = torch.tensor([[5, 5], [1, 2], [3, 4]])  # t, h, w for two tokens
    r = ernie_3d_angles(pos, 16, 10000.0, 2)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16))
    expect0 = torch.tensor([1, 3, 1, 3, 1, 3, 5, 5]).float() * inv  # h, w alternate; last two follow t
    assert torch.allclose(r.freqs[0], expect0)
    assert torch.allclose(r.freqs[1], torch.tensor([2, 4, 2, 4, 2, 4, 5, 5]).float() * inv)


def test_tiny_ernie_vl_routes_by_modality():
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-ernie-vl")
    torch.manual_seed(0)
    model = build_model(cfg)
    T = 24
    tokens = torch.randint(0, cfg.vocab_size, (T,))
    pos3 = torch.stack([torch.arange(T)] * 3)
    tt = torch.zeros(T, dtype=torch.long)
    tt[8:16] = 1
    loss = model(tokens, pos3, labels=torch.roll(tokens, -1), loss_mask=torch.ones(T), token_type=tt).mean()
    loss.backward()
    moe = model.decoder.layers[1].mlp
    assert moe.text.experts.linear_fc1.weights()[0].shape[0] == 2 * 32
    assert moe.vision.experts.linear_fc1.weights()[0].shape[0] == 2 * 16
    assert all(p.grad is not None for p in model.parameters())
    # text-only batch: vision experts receive no tokens but the step still runs
    model.zero_grad()
    model(tokens, pos3, labels=torch.roll(tokens, -1), loss_mask=torch.ones(T), token_type=torch.zeros(T, dtype=torch.long)).mean().backward()
    g = moe.vision.experts.linear_fc1.weights()[0].grad
    assert g is None or float(g.abs().sum()) == 0.0

