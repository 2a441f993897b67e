"""Tiny Llama-style decoder on CPU/gloo: pure data parallel (world 2), 20 Adam steps, then a
torch_dist checkpoint round trip with bit-identical continuation; plus single-process parity
against an independent plain-PyTorch implementation of the same model."""
import math
import os
import tempfile

import pytest
import torch

from dist_utils import run_distributed


def _tiny_cfg():
    from loongforge_b200.models.registry import get_model_config

    return get_model_config("tiny-llama")


def _make_trainer(world_dp, train_iters=20, gbs=4, **kw):
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    tc = TrainConfig(micro_batch_size=2, global_batch_size=gbs, seq_length=128, train_iters=train_iters, lr=1e-4,
                     weight_decay=0.0, clip_grad=0.0, log_interval=1000, **kw)
    return Trainer(_tiny_cfg(), tc)


def _dp2_worker(rank, world, tmp):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator

    tr = _make_trainer(world)
    st = tr.st
    assert st.dp_size == 2
    it = synthetic_batch_iterator(32000, 128, 2, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=7, pin_memory=False)
    losses = [tr.train_step(it)["lm loss"] for _ in range(20)]
    tr.save_checkpoint(tmp)
    cont = tr.train_step(it)["lm loss"]
    # fresh trainer, reload, same data position -> identical loss
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    tr2 = _make_trainer(world)
    assert tr2.load_checkpoint(tmp) == 20
    it2 = synthetic_batch_iterator(32000, 128, 2, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=7, pin_memory=False,
                                   start_sample=tr2.consumed_samples)
    again = tr2.train_step(it2)["lm loss"]
    return losses, cont, again


def test_dp2_train_and_bit_identical_resume():
    with tempfile.TemporaryDirectory() as tmp:
        res = run_distributed(_dp2_worker, 2, tmp)
        files = os.listdir(os.path.join(tmp, "iter_0000020"))
        assert "metadata.json" in files and "common.pt" in files and ".metadata" in files
        assert any(f.endswith(".distcp") for f in files)
        assert open(os.path.join(tmp, "latest_checkpointed_iteration.txt")).read().strip() == "20"
    (l0, c0, a0), (l1, c1, a1) = res
    assert l0 == l1, "data-parallel ranks must report the same averaged loss"
    assert abs(l0[0] - math.log(32000)) < 0.2
    assert l0[-1] < l0[0]
    assert c0 == a0 and c1 == a1, f"resume is not bit-identical: {c0} vs {a0}"


class _RefLlama(torch.nn.Module):
    """Independent reference: plain PyTorch ops, HF-style separate q/k/v and gate/up weights."""

    def __init__(self, model):
        super().__init__()
        self.m = model
        self.cfg = model.cfg

    def forward(self, tokens, labels):
        cfg = self.cfg
        m = self.m
        B, S = tokens.shape
        x = m.embedding.word_embeddings.weight[tokens]
        d, nq, ng = cfg.kv_channels, cfg.num_attention_heads, cfg.num_query_groups
        r = nq // ng
        inv = 1.0 / (cfg.rotary_base ** (torch.arange(0, d, 2).float() / d))
        ang = torch.outer(torch.arange(S).float(), inv)
        cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

        def rope(t):
            a, b = t[..., : d // 2], t[..., d // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

        def norm(t, w):
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.layernorm_epsilon) * w

        for layer in m.decoder.layers:
            att = layer.self_attention
            h = norm(x, att.linear_qkv.layer_norm_weight)
            qkv = (h @ att.linear_qkv.weight.t()).view(B, S, ng, r + 2, d)
            q = rope(qkv[:, :, :, :r].reshape(B, S, nq, d))
            k = rope(qkv[:, :, :, r])
            v = qkv[:, :, :, r + 1]
            k = k.repeat_interleave(r, 2)
            v = v.repeat_interleave(r, 2)
            s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(d)
            s = s.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool)), float("-inf"))
            o = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v).reshape(B, S, nq * d)
            x = x + o @ att.linear_proj.weight.t()
            h = norm(x, layer.mlp.linear_fc1.layer_norm_weight)
            gu = h @ layer.mlp.linear_fc1.weight.t()
            g, u = gu.chunk(2, -1)
            x = x + (torch.nn.functional.silu(g) * u) @ layer.mlp.linear_fc2.weight.t()
        x = norm(x, m.decoder.final_layernorm.weight)
        logits = x @ m.output_layer.weight.t()
        return torch.nn.functional.cross_entropy(logits.view(B * S, -1)[:, : cfg.vocab_size], labels.reshape(-1))


def test_model_matches_independent_reference():
    from loongforge_b200.models.gpt import GPTModel

    torch.manual_seed(0)
    cfg = _tiny_cfg()
    model = GPTModel(cfg)
    B, S = 2, 64
    tokens = torch.randint(0, cfg.vocab_size, (B, S))
    labels = torch.randint(0, cfg.vocab_size, (B, S))
    pos = torch.arange(S).repeat(B)
    from loongforge_b200.models.transformer import PackedSeqParams

    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32)
    losses = model(tokens.reshape(-1), pos, labels=labels.reshape(-1), loss_mask=torch.ones(B * S),
                   packed=PackedSeqParams(cu_seqlens=cu, max_seqlen=S))
    loss = losses.mean()
    loss.backward()
    g_ours = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    ref = _RefLlama(model)(tokens, labels)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    for n, p in model.named_parameters():
        assert torch.allclose(g_ours[n], p.grad, atol=2e-5, rtol=1e-3), n


def test_master_remainder_is_exact_fp32():
    """(bf16, int16 remainder) reproduces the fp32 master bit for bit, and AdamW on it equals AdamW on fp32."""
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(0)
    master = torch.randn(10001) * torch.logspace(-6, 3, 10001)
    w = torch.empty(10001, dtype=torch.bfloat16)
    lo = torch.empty(10001, dtype=torch.int16)
    OF.master_split(master, w, lo)
    assert torch.equal(OF.master_join(w, lo), master)
    assert torch.equal(w, master.to(torch.bfloat16))
    g = torch.randn(10001)
    m1, v1 = torch.zeros(10001), torch.zeros(10001)
    m2, v2 = torch.zeros(10001), torch.zeros(10001)
    ref = master.clone()
    for step in (1, 2, 3):
        OF.adam_step(ref, g, m1, v1, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        OF.adam_step_remainder(w, lo, g, m2, v2, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    assert torch.equal(OF.master_join(w, lo), ref)


def _async_worker(rank, world, tmp):
    from loongforge_b200.ckpt import checkpointing
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.parallel import state as ps

    tr = _make_trainer(world, async_save=True)
    st = tr.st
    it = synthetic_batch_iterator(32000, 128, 2, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=7, pin_memory=False)
    for _ in range(3):
        tr.train_step(it)
    tr.save_checkpoint(tmp)
    tracker_before = os.path.exists(os.path.join(tmp, "latest_checkpointed_iteration.txt"))
    nxt = tr.train_step(it)["lm loss"]  # training continues while the write is in flight
    checkpointing.finalize_async_save(tr)
    tracker_after = open(os.path.join(tmp, "latest_checkpointed_iteration.txt")).read().strip()
    ps.destroy_model_parallel()
    tr2 = _make_trainer(world)
    assert tr2.load_checkpoint(tmp) == 3
    it2 = synthetic_batch_iterator(32000, 128, 2, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=7, pin_memory=False,
                                   start_sample=tr2.consumed_samples)
    return tracker_before, tracker_after, nxt, tr2.train_step(it2)["lm loss"]


def test_async_save_publishes_tracker_after_the_write():
    with tempfile.TemporaryDirectory() as tmp:
        for before, after, nxt, again in run_distributed(_async_worker, 2, tmp):
            assert before is False and after == "3"
            assert nxt == again  # the checkpoint holds the state at save time, not the later step's


def test_dynamic_ntk_rotary_base_grows_beyond_the_trained_context():
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.models.gpt import RotaryEmbedding

    cfg = TransformerConfig(max_position_embeddings=128, rotary_dynamic_ntk=True, rotary_dynamic_ntk_factor=8.0)
    rot = RotaryEmbedding(cfg, 64)
    short, long = rot.table(128, "cpu").freqs, rot.table(512, "cpu").freqs
    plain = RotaryEmbedding(TransformerConfig(max_position_embeddings=128), 64).table(512, "cpu").freqs
    assert torch.equal(short, plain[:128]), "within the trained context nothing changes"
    base = 10000.0 * ((8.0 * 512 / 128) - 7.0) ** (64 / 62)
    want = torch.outer(torch.arange(512.0), 1.0 / base ** (torch.arange(0, 64, 2).float() / 64))
    assert torch.allclose(long, want, rtol=1e-5) and not torch.allclose(long, plain)
