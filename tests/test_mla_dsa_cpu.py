"""Multi-latent attention with the sparse-attention indexer (DeepSeek-V3.2 path) on CPU."""
import torch


def test_sparse_mla_with_all_keys_selected_is_dense_causal_attention():
    from loongforge_b200.ops import dsa_ops

    torch.manual_seed(0)
    T, H, Dk, dv = 20, 3, 24, 16
    q = torch.randn(T, H, Dk, requires_grad=True)
    kv = torch.randn(T, Dk, requires_grad=True)
    idx = torch.arange(T).unsqueeze(0).expand(T, T).clone()
    idx[torch.triu(torch.ones(T, T, dtype=torch.bool), 1)] = -1  # causal: keys after the query are empty slots
    o, pmean = dsa_ops.sparse_mla_attention(q, kv, idx, 0.2, d_v=dv, block=7, return_head_mean_probs=True)
    s = torch.einsum("thd,sd->ths", q, kv) * 0.2
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1).unsqueeze(1), float("-inf"))
    p = s.softmax(-1)
    ref = torch.einsum("ths,sd->thd", p, kv[:, :dv])
    assert torch.allclose(o, ref, atol=1e-5) and torch.allclose(pmean, p.mean(1), atol=1e-6)
    w = torch.randn_like(ref)
    ga = torch.autograd.grad((o * w).sum(), [q, kv])
    gb = torch.autograd.grad((ref * w).sum(), [q, kv])
    for a, b in zip(ga, gb):
        assert torch.allclose(a, b, atol=1e-5)


def test_indexer_topk_is_causal_and_picks_best():
    from loongforge_b200.ops import dsa_ops

    torch.manual_seed(1)
    T, Hi, D, k = 30, 2, 8, 4
    q, kk, w = torch.randn(T, Hi, D), torch.randn(T, D), torch.rand(T, Hi)
    pos = torch.arange(T)
    idx, sc = dsa_ops.indexer_topk(q, kk, w, k, pos, pos, block=11)
    full = dsa_ops.indexer_logits_block(q, kk, w).masked_fill(pos[None, :] > pos[:, None], float("-inf"))
    for t in range(T):
        sel = [i for i in idx[t].tolist() if i >= 0]
        assert all(i <= t for i in sel) and len(sel) == min(k, t + 1)
        assert set(sel) == set(full[t].topk(len(sel)).indices.tolist())
    at = dsa_ops.indexer_scores_at(q, w, kk, idx, block=9)
    assert torch.allclose(at[idx >= 0], sc[idx >= 0], atol=1e-5)


def test_tiny_deepseek_v32_trains_with_indexer_loss():
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-deepseek")
    assert cfg.use_dsa and cfg.multi_latent_attention and cfg.dsa_indexer_loss_coeff > 0
    torch.manual_seed(0)
    model = build_model(cfg)
    model.train()
    opt = torch.optim.AdamW(model.parameters(), lr=2e-3)
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
    idx_params = [n for n, p in model.named_parameters() if ".indexer." in n]
    assert idx_params and all(p.grad is not None and float(p.grad.abs().sum()) > 0
                              for n, p in model.named_parameters() if ".indexer." in n)  # trained by the KL loss
    assert all(p.grad is not None for p in model.parameters())
    assert losses[-1] < losses[0] - 0.2, losses


def test_index_share_layers_reuse_topk_and_train():
    """GLM-5.2 IndexShare: with frequency 4 and offset 3 the layers 0, 1, 2, 6, 10, ... own an indexer; the others
    take the indices of the latest computing layer, also when activations are recomputed."""
    import torch

    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps

    c = TransformerConfig(num_layers=78, dsa_indexer_topk_freq=4, dsa_indexer_skip_topk_offset=3)
    owners = [l for l in range(78) if c.dsa_computes_topk(l)]
    assert owners[:6] == [0, 1, 2, 6, 10, 14] and owners[-1] == 74 and len(owners) == 21
    assert [c.dsa_source_layer(l) for l in (3, 5, 6, 9, 77)] == [2, 2, 6, 6, 74]
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-glm")  # 6 layers, frequency 2, offset 1 -> layers 0, 2, 4 compute
    model = build_model(cfg)
    has = [hasattr(l.self_attention.core_attention, "indexer") for l in model.decoder.layers]
    assert has == [True, False, True, False, True, False]
    T = 48
    tok = torch.randint(0, cfg.vocab_size, (T,))
    out = {}
    for rec in (None, "full"):
        cfg.recompute_granularity = rec
        model.zero_grad()
        model(tok, torch.arange(T), labels=torch.roll(tok, -1), loss_mask=torch.ones(T)).mean().backward()
        idx = [l.self_attention.last_topk_indices for l in model.decoder.layers]
        assert torch.equal(idx[1], idx[0]) and torch.equal(idx[3], idx[2]) and not torch.equal(idx[2], idx[0])
        out[rec] = model.decoder.layers[1].self_attention.linear_proj.weight.grad.clone()
    assert torch.allclose(out[None], out["full"], atol=1e-6), "recomputation sees the same shared indices"
    # a pipeline stage may not start on a layer that reuses indices
    from loongforge_b200.models.gpt import GPTModel
    import pytest
    with pytest.raises(ValueError, match="IndexShare"):
        GPTModel(cfg, pre_process=False, post_process=True, layer_numbers=[3, 4, 5])


def test_sparse_mla_block_backward_from_saved_lse_matches_autograd():
    """The GEMM formulation of the sparse attention backward (from output + log-sum-exp, no autograd graph) against
    autograd through the gather formulation: ragged selections, an empty row, repeated keys across queries."""
    import torch

    from loongforge_b200.ops import dsa_ops as D

    torch.manual_seed(0)
    m, H, n, K, scale = 12, 8, 50, 16, 0.07
    q = torch.randn(m, H, 576, requires_grad=True)
    kv = torch.randn(n, 576, requires_grad=True)
    idx = torch.stack([torch.randperm(n)[:K] for _ in range(m)])
    idx[0] = -1
    idx[3, 5:] = -1
    do = torch.randn(m, H, 512)
    o = D._sparse_mla_block(q, idx, kv, scale, 512, False).view(m, H, 512)
    o.backward(do)
    g = kv.detach()[idx.clamp_min(0)]
    sc = torch.einsum("bhd,bkd->bhk", q.detach(), g) * scale
    lse = torch.logsumexp(sc.masked_fill(~(idx >= 0)[:, None, :], float("-inf")), -1)
    dkv = torch.zeros(n, 576)
    dq = torch.cat([D.sparse_mla_backward_block(q.detach()[s:s + 5], kv.detach(), idx[s:s + 5], o.detach()[s:s + 5],
                                                lse[s:s + 5], do[s:s + 5], scale, dkv) for s in range(0, m, 5)])
    assert torch.allclose(dq, q.grad, atol=2e-5) and torch.allclose(dkv, kv.grad, atol=2e-5)
    assert dq[0].abs().max() == 0
