"""ChunkPipe gradients equal those of the un-chunked sequence; balanced group sampler and savable iterators."""
import pytest
import torch

from loongforge_b200.runtime import chunkpipe as CP


def _grads(model_parts):
    return [p.grad.clone() for m in model_parts for p in m.parameters()]


def test_chunkpipe_matches_full_sequence():
    torch.manual_seed(0)
    dim, T, V = 32, 50, 64
    layers = torch.nn.ModuleList([CP.CausalSelfAttentionBlock(dim, 4) for _ in range(3)])
    emb, head = torch.nn.Embedding(V, dim), torch.nn.Linear(dim, V)
    tokens = torch.randint(0, V, (T,))
    labels = torch.roll(tokens, -1)

    def loss_fn(h, s, e):
        return torch.nn.functional.cross_entropy(head(h), labels[s:e], reduction="sum") / T

    x = emb(tokens)
    for layer in layers:
        x, _ = layer(x, None, 0)
    ref = loss_fn(x, 0, T)
    ref.backward()
    want = _grads([layers, emb, head])
    for m in (layers, emb, head):
        m.zero_grad()
    got_loss = CP.chunkpipe_forward_backward(layers, emb, loss_fn, tokens, num_chunks=4)
    assert abs(got_loss - float(ref)) < 1e-4
    for a, b in zip(_grads([layers, emb, head]), want):
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-4), (a - b).abs().max()
    assert CP.chunk_bounds(50, 4) == [(0, 13), (13, 26), (26, 39), (39, 50)]
    assert CP.num_microbatches_with_chunks(8, 4) == 32


def test_balanced_group_sampler_and_savable_iterator():
    from loongforge_b200.data.samplers import BalancedGroupSampler, SavableCyclicIterator

    lengths = [4000, 100, 200, 3900, 150, 50, 3000, 2900] * 4
    samplers = [BalancedGroupSampler(lengths, 8, 2, r, capacity=4096, seed=1) for r in range(2)]
    its = [iter(s) for s in samplers]
    for _ in range(3):
        shares = [next(it) for it in its]
        flat = [[i for p in sh for i in p] for sh in shares]
        assert len(set(flat[0]) | set(flat[1])) == 8 and not set(flat[0]) & set(flat[1])
        cost = [sum(lengths[i] ** 2 for i in f) for f in flat]
        assert max(cost) / (sum(cost) / 2) < 1.25
        for sh in shares:
            assert all(sum(min(lengths[i], 4096) for i in p) <= 4096 for p in sh)
    sd = samplers[0].state_dict()
    nxt = next(its[0])
    s2 = BalancedGroupSampler(lengths, 8, 2, 0, capacity=4096, seed=1)
    s2.load_state_dict(sd)
    assert next(iter(s2)) == nxt
    it = SavableCyclicIterator(list(range(5)), seed=3)
    first = [next(it) for _ in range(7)]
    assert sorted(first[:5]) == [0, 1, 2, 3, 4]
    sd = it.state_dict()
    a = [next(it) for _ in range(4)]
    it2 = SavableCyclicIterator(list(range(5)), seed=3)
    it2.load_state_dict(sd)
    assert [next(it2) for _ in range(4)] == a


@pytest.mark.parametrize("model_name", ["tiny-llama", "tiny-qwen3-moe"])
def test_trainer_with_chunk_pipelining_matches_whole_sequences(model_name):
    """The trainer's chunk-pipelined step (4 chunks per sequence, keys / values of earlier chunks as attention
    prefix, gradients across chunks through the caches) reproduces the ordinary step's losses and gradient norms."""
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    def run(chunks):
        ps.destroy_model_parallel()
        cfg = get_model_config(model_name, moe_aux_loss_coeff=0.0) if "moe" in model_name else get_model_config(model_name)
        tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=64, train_iters=3, lr=1e-3,
                         log_interval=1000, chunkpipe_chunks=chunks)
        tr = Trainer(cfg, tc)
        it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, seed=4, pin_memory=False)
        return [(m["lm loss"], m["grad_norm"]) for m in (tr.train_step(it) for _ in range(3))]

    ref, got = run(0), run(4)
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) < 1e-4 * max(1, abs(l0)) and abs(g0 - g1) < 1e-3 * max(1, abs(g0)), (ref, got)


def _chunk_tp(rank, world, chunks, dims_kw, sp):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-qwen3-moe", moe_aux_loss_coeff=0.0)
    cfg.sequence_parallel = sp and dims_kw.get("tp", 1) > 1
    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=64, train_iters=2, lr=1e-3, log_interval=1000,
                     chunkpipe_chunks=chunks)
    tr = Trainer(cfg, tc, ParallelDims(**dims_kw))
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, seed=4, pin_memory=False)
    return [(m["lm loss"], m["grad_norm"]) for m in (tr.train_step(it) for _ in range(2))]


@pytest.mark.parametrize("sp", [True, False])
def test_chunk_pipelining_under_tensor_parallelism(sp):
    from dist_utils import run_distributed

    ref = run_distributed(_chunk_tp, 1, 0, {}, False)[0]
    got = run_distributed(_chunk_tp, 2, 4, {"tp": 2}, sp)[0]
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) < 1e-4 * abs(l0) and abs(g0 - g1) < 1e-3 * max(1, g0), (ref, got)


def _chunk_pp(rank, world, chunks, dims_kw):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-llama", num_layers=4)
    cfg.sequence_parallel = dims_kw.get("tp", 1) > 1
    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=64, train_iters=2, lr=1e-3, log_interval=1000,
                     chunkpipe_chunks=chunks, clip_grad=1.0)
    tr = Trainer(cfg, tc, ParallelDims(**dims_kw))
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, seed=4, pin_memory=False)
    return [(m.get("lm loss"), m["grad_norm"]) for m in (tr.train_step(it) for _ in range(2))]


@pytest.mark.parametrize("dims,world", [({"pp": 2}, 2), ({"pp": 2, "tp": 2}, 4)])
def test_chunks_flow_through_pipeline_stages(dims, world):
    """Chunk pipelining with pipeline parallelism: every stage keeps the K/V caches of its layers, chunks travel between
    stages like micro-batches (forward in order, backward in reverse); same trajectory as whole sequences on one rank."""
    from dist_utils import run_distributed

    ref = run_distributed(_chunk_pp, 1, 0, {})[0]
    got = run_distributed(_chunk_pp, world, 4, dict(dims))
    last = got[world - 1]  # a rank of the last stage reports the loss
    for (l0, g0), (l1, g1) in zip(ref, last):
        assert l1 is not None and abs(l0 - l1) < 1e-4 * abs(l0) and abs(g0 - g1) < 1e-3 * max(1, g0), (ref, got)
    for (_, g0), (_, g1) in zip(ref, got[0]):
        assert abs(g0 - g1) < 1e-3 * max(1, g0)  # the global gradient norm is the same on every stage


@pytest.mark.parametrize("use_dsa", [True, False])
def test_chunk_pipelining_with_multi_latent_attention(use_dsa):
    """MLA under chunk pipelining: the sparse form caches compressed keys and indexer keys per chunk (top-k selection over
    prefix + chunk), the dense form the materialised keys / values; same trajectory as whole sequences."""
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    def run(chunks):
        ps.destroy_model_parallel()
        cfg = get_model_config("tiny-deepseek", moe_aux_loss_coeff=0.0, use_dsa=use_dsa)
        tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=64, train_iters=2, lr=1e-3,
                         log_interval=1000, chunkpipe_chunks=chunks)
        tr = Trainer(cfg, tc)
        it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, seed=4, pin_memory=False)
        return [(m["lm loss"], m["grad_norm"]) for m in (tr.train_step(it) for _ in range(2))]

    ref, got = run(0), run(4)
    ps.destroy_model_parallel()
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) < 2e-4 * max(1, abs(l0)) and abs(g0 - g1) < 2e-3 * max(1, abs(g0)), (ref, got)
