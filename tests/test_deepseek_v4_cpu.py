"""DeepSeek-V4 pieces: sparse MQA with sink, window/compressed index rules, hyper-connections, hash routing,
and a tiny end-to-end model."""
import torch


def test_sparse_mqa_with_sink_matches_dense_softmax():
    from loongforge_b200.models.csa import sparse_mqa_attention_with_sink, window_indices

    torch.manual_seed(0)
    T, H, d = 12, 3, 8
    q, kv = torch.randn(T, H, d), torch.randn(T, d)
    sink = torch.randn(H)
    idx = window_indices(T, T, None, "cpu")  # full causal window
    out = sparse_mqa_attention_with_sink(q, kv, idx, sink, 0.3)
    s = torch.einsum("thd,sd->ths", q, kv) * 0.3
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1).unsqueeze(1), float("-inf"))
    full = torch.cat([s, sink.view(1, H, 1).expand(T, H, 1)], -1).softmax(-1)[..., :T]
    assert torch.allclose(out, torch.einsum("ths,sd->thd", full, kv), atol=1e-5)


def test_window_and_compressed_entries_are_causal_and_sequence_local():
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.models.csa import Compressor, CSAIndexer, window_indices

    cu = [0, 10, 23]
    idx = window_indices(23, 4, cu, "cpu")
    assert idx[0].tolist() == [0, -1, -1, -1] and idx[10].tolist() == [10, -1, -1, -1]
    assert idx[12].tolist() == [12, 11, 10, -1] and idx[22].tolist() == [22, 21, 20, 19]
    cfg = TransformerConfig(hidden_size=16, num_attention_heads=2, dsa_indexer_n_heads=2, dsa_indexer_head_dim=8,
                            dsa_indexer_topk=3)
    torch.manual_seed(0)
    comp = Compressor(cfg, "c", 4, 8)
    x, kv = torch.randn(23, 16), torch.randn(23, 8)
    entries, ends, starts = comp(x, kv, cu)
    assert entries.shape == (2 + 3, 8)
    assert ends.tolist() == [3, 7, 13, 17, 21] and starts.tolist() == [0, 0, 10, 10, 10]
    token_start = torch.tensor([0] * 10 + [10] * 13)
    sel = CSAIndexer(cfg, "i", 8)(x, entries, ends, starts, token_start)
    for t in range(23):
        for j in sel[t].tolist():
            if j >= 0:
                assert ends[j] <= t and starts[j] == token_start[t]
    assert (sel[:3] == -1).all() and (sel[22] >= 0).sum() == 3


def test_hyper_connection_starts_as_plain_residual_and_sinkhorn_is_doubly_stochastic():
    from loongforge_b200.models.hyper_connections import HyperConnection, sinkhorn

    m = sinkhorn(torch.randn(5, 4, 4), 30)
    assert torch.allclose(m.sum(-1), torch.ones(5, 4), atol=1e-3) and torch.allclose(m.sum(-2), torch.ones(5, 4), atol=1e-3)
    hc = HyperConnection(8, 4, 20, 0.0, 1e-6, "k")  # zero gate: maps are the static base
    xs = torch.randn(6, 1, 8).expand(6, 4, 8).contiguous()
    h, maps = hc.read(xs)
    assert torch.allclose(h, 2.0 * xs[:, 0], atol=1e-5)  # 4 streams x sigmoid(0)
    out = hc.write(xs, torch.ones(6, 8), maps)
    assert torch.allclose(out, xs + 1.0, atol=2e-2)  # near-identity mixing, write weight 1


def test_hash_routing_is_deterministic_and_distinct():
    from loongforge_b200.ops.moe_ops import hash_routing

    ids = torch.randint(0, 50000, (200,))
    a, b = hash_routing(ids, 64, 6), hash_routing(ids, 64, 6)
    assert torch.equal(a, b) and a.min() >= 0 and a.max() < 64
    assert all(len(set(r)) == 6 for r in a.tolist())
    assert len(set(a[:, 0].tolist())) > 20  # spreads over experts


def test_tiny_deepseek_v4_trains():
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-deepseek-v4")
    torch.manual_seed(0)
    model = build_model(cfg)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    T = 48
    tokens = torch.randint(0, cfg.vocab_size, (T,))
    labels, pos = torch.roll(tokens, -1), torch.arange(T)
    losses = []
    for _ in range(8):
        loss = model(tokens, pos, labels=labels, loss_mask=torch.ones(T)).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert all(".indexer." in n for n in missing), missing  # the selection itself is not differentiable
    assert losses[-1] < losses[0] - 0.3, losses


def test_clamped_swiglu():
    from loongforge_b200.models.transformer import clamped_swiglu

    h = torch.tensor([[20.0, -3.0, 50.0, -50.0]])  # gate = [20, -3], up = [50, -50]
    out = clamped_swiglu(h, 10.0)
    assert torch.allclose(out, torch.stack([torch.nn.functional.silu(torch.tensor(10.0)) * 10.0,
                                            torch.nn.functional.silu(torch.tensor(-3.0)) * -10.0]).view(1, 2))


def test_blockwise_apply_matches_plain_autograd():
    from loongforge_b200.models.csa import sparse_mqa_attention_with_sink
    from loongforge_b200.ops.blockwise import blockwise_apply

    torch.manual_seed(0)
    T, H, d, K = 37, 3, 8, 6
    q = torch.randn(T, H, d, requires_grad=True)
    kv = torch.randn(T, d, requires_grad=True)
    sink = torch.randn(H, requires_grad=True)
    idx = torch.randint(-1, T, (T, K))
    ref = sparse_mqa_attention_with_sink(q, kv, idx, sink, 0.3)
    w = torch.randn_like(ref)
    g_ref = torch.autograd.grad((ref * w).sum(), [q, kv, sink])
    out = blockwise_apply(lambda qb, ib, kvv, sk: sparse_mqa_attention_with_sink(qb, kvv, ib, sk, 0.3), [q, idx],
                          [kv, sink], block=8)
    g = torch.autograd.grad((out * w).sum(), [q, kv, sink])
    assert torch.allclose(out, ref, atol=1e-6)
    for a, b in zip(g, g_ref):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
