"""Megatron-facing parallel API: RNG tracker + RNG-exact checkpointing, broadcast_data, FSDP2 wrapping."""
import torch

from tests.dist_utils import run_distributed


def test_rng_tracker_fork_and_seed_rules():
    from loongforge_b200.parallel import random as R

    R.model_parallel_manual_seed(1234, tp_rank=0)
    with R.get_rng_tracker().fork():
        a0 = torch.rand(4)
    d0 = torch.rand(4)
    R.model_parallel_manual_seed(1234, tp_rank=1)
    with R.get_rng_tracker().fork():
        a1 = torch.rand(4)
    d1 = torch.rand(4)
    assert torch.equal(d0, d1) and not torch.equal(a0, a1)  # default stream equal across TP, forked stream differs
    tr = R.get_rng_tracker()
    before = tr.get_states()[R.MODEL_PARALLEL_RNG].clone()
    with tr.fork():
        torch.rand(1)
    assert not torch.equal(before, tr.get_states()[R.MODEL_PARALLEL_RNG])


def test_checkpoint_replays_dropout_exactly():
    from loongforge_b200.parallel import random as R

    R.model_parallel_manual_seed(7)
    w = torch.randn(16, 16, requires_grad=True)

    def block(x):
        with R.get_rng_tracker().fork():
            h = torch.nn.functional.dropout(x @ w, 0.5, training=True)
        return torch.nn.functional.dropout(h.relu(), 0.3, training=True)

    x = torch.randn(8, 16, requires_grad=True)
    R.model_parallel_manual_seed(7)
    y = block(x)
    y.sum().backward()
    gw, gx = w.grad.clone(), x.grad.clone()
    w.grad = x.grad = None
    R.model_parallel_manual_seed(7)
    y2 = R.checkpoint(block, x)
    torch.rand(100)  # consume randomness between forward and backward: the replay must not be affected
    y2.sum().backward()
    assert torch.equal(y, y2) and torch.allclose(gw, w.grad) and torch.allclose(gx, x.grad)


def _bcast(rank, world):
    import torch.distributed as dist
    from loongforge_b200.parallel.data import broadcast_data, broadcast_flags

    data = {"tokens": torch.arange(12).view(3, 4), "labels": torch.arange(5), "none": None} if rank == 0 else None
    out = broadcast_data(["tokens", "labels", "none"], data, torch.long, dist.group.WORLD, 0)
    return out["tokens"].tolist(), out["labels"].tolist(), out["none"], broadcast_flags(3 if rank == 0 else 0, dist.group.WORLD, 0)


def test_broadcast_data():
    for r in run_distributed(_bcast, 2):
        assert r == ([[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11]], [0, 1, 2, 3, 4], None, 3)


def _fsdp(rank, world):
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.parallel.fsdp import full_state_dict, wrap_fsdp2

    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-llama", vocab_size=512)
    cfg.gradient_accumulation_fusion = False
    torch.manual_seed(0)
    ref = build_model(cfg)
    model = build_model(cfg)
    model.load_state_dict(ref.state_dict())
    wrap_fsdp2(model)
    T = 32
    torch.manual_seed(100 + rank)
    tokens = torch.randint(0, 512, (T,))
    args = (tokens, torch.arange(T))
    kw = dict(labels=torch.roll(tokens, -1), loss_mask=torch.ones(T))
    model(*args, **kw).mean().backward()
    sharded = model.decoder.layers[0].mlp.linear_fc2.weight
    local_rows = sharded.to_local().shape[0]
    # reference: average of both ranks' gradients, computed locally on the un-sharded copy
    g = None
    for r in range(world):
        torch.manual_seed(100 + r)
        tk = torch.randint(0, 512, (T,))
        ref.zero_grad()
        ref(tk, torch.arange(T), labels=torch.roll(tk, -1), loss_mask=torch.ones(T)).mean().backward()
        gi = ref.decoder.layers[0].mlp.linear_fc2.weight.grad.clone()
        g = gi if g is None else g + gi
    err = (sharded.grad.full_tensor() - g / world).abs().max().item()
    return local_rows, sharded.shape[0], err, len(full_state_dict(model))


def test_fsdp2_wrapping_shards_and_matches_dp_average():
    res = run_distributed(_fsdp, 2)
    for local_rows, rows, err, n in res:
        assert local_rows == rows // 2 and err < 1e-5 and n > 10


def _hetero(rank, world):
    import torch.distributed as dist
    from loongforge_b200.runtime.hetero_dp import FullHeteroEncoderRunner, owner_of, rounds

    torch.manual_seed(0)
    enc = torch.nn.Linear(6, 4)
    inputs = [torch.randn(3 + i, 6) for i in range(5)]  # 5 micro-batches, identical on both ranks
    calls = []

    def encode(x):
        calls.append(x.shape[0])
        return enc(x)

    runner = FullHeteroEncoderRunner(dist.group.WORLD, encode)
    embs = runner.encode_all(inputs)
    # the "language model": both ranks compute the same loss; only rank 0 contributes its gradient
    loss = sum((e * (i + 1)).sum() for i, e in enumerate(embs))
    loss.backward()
    runner.backward(contributes=(rank == 0))
    g = enc.weight.grad.clone()
    dist.all_reduce(g)  # owners hold disjoint parts of the encoder gradient: DP all-reduce completes it
    ref = torch.nn.Linear(6, 4)
    ref.load_state_dict(enc.state_dict())
    sum((ref(x) * (i + 1)).sum() for i, x in enumerate(inputs)).backward()
    assert owner_of(3, 2) == 1 and rounds(5, 2) == 3
    return calls, float((g - ref.weight.grad).abs().max()), [tuple(e.shape) for e in embs]


def test_full_hetero_encoder_runner():
    res = run_distributed(_hetero, 2)
    assert res[0][0] == [3, 5, 7] and res[1][0] == [4, 6]  # each rank encoded only its own micro-batches
    for calls, err, shapes in res:
        assert err < 1e-5 and shapes == [(3, 4), (4, 4), (5, 4), (6, 4), (7, 4)]
