"""TP / SP / PP / EP / DP layouts on CPU (gloo) must reproduce the single-process training
trajectory of the same model and data (same global batch, same seed)."""
import pytest
import torch

from dist_utils import run_distributed


def _run(rank, world, model_name, dims_kw, steps, overrides, gbs=4, mbs=1):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config(model_name, **overrides)
    if dims_kw.get("tp", 1) > 1:
        cfg.sequence_parallel = dims_kw.pop("sp", True)
    dims_kw.pop("sp", None)
    tc = TrainConfig(micro_batch_size=mbs, global_batch_size=gbs, seq_length=64, train_iters=steps, lr=1e-3,
                     clip_grad=1.0, log_interval=1000)
    tr = Trainer(cfg, tc, ParallelDims(**dims_kw))
    st = tr.st
    it = synthetic_batch_iterator(cfg.vocab_size, 64, mbs, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=3,
                                  pin_memory=False)
    out = []
    for _ in range(steps):
        m = tr.train_step(it)
        out.append((m.get("lm loss"), m["grad_norm"]))
    return out


_REF = {}


def _single(model_name, steps, overrides, gbs=4, mbs=1):
    """Single-process reference trajectory; computed once per configuration and test process."""
    key = (model_name, steps, repr(sorted(overrides.items())), gbs, mbs)
    if key not in _REF:
        _REF[key] = run_distributed(_run, 1, model_name, {}, steps, overrides, gbs, mbs)[0]
    return _REF[key]


def _check(ref, res, have_loss, tol=2e-4):
    for r, got in enumerate(res):
        for (l0, g0), (l1, g1) in zip(ref, got):
            if have_loss(r):
                assert l1 is not None and abs(l0 - l1) < tol * max(1, abs(l0)), (r, l0, l1)
            assert abs(g0 - g1) < 5e-4 * max(1, abs(g0)), (r, g0, g1)


@pytest.mark.parametrize("dims,world", [({"tp": 2}, 2), ({"tp": 2, "sp": False}, 2), ({"pp": 2}, 2),
                                        ({"tp": 2, "pp": 2}, 4)])
def test_dense_layouts_match_single_process(dims, world):
    ref = _single("tiny-llama", 3, {})
    res = run_distributed(_run, world, "tiny-llama", dict(dims), 3, {})
    pp = dims.get("pp", 1)
    tp = dims.get("tp", 1)
    _check(ref, res, lambda r: r // (world // pp) == pp - 1)


def test_moe_expert_parallel_matches_single_process():
    ov = {"moe_aux_loss_coeff": 0.0}
    ref = _single("tiny-qwen3-moe", 3, ov)
    res = run_distributed(_run, 2, "tiny-qwen3-moe", {"ep": 2}, 3, ov)
    _check(ref, res, lambda r: True, tol=5e-4)


def test_moe_expert_tensor_parallel_matches_single_process():
    """Experts sliced over the expert-tensor-parallel group (= the TP ranks), tokens sequence parallel."""
    ov = {"moe_aux_loss_coeff": 0.0}
    ref = _single("tiny-qwen3-moe", 3, ov)
    res = run_distributed(_run, 2, "tiny-qwen3-moe", {"tp": 2, "etp": 2}, 3, ov)
    _check(ref, res, lambda r: True, tol=5e-4)


@pytest.mark.parametrize("model,dims", [("tiny-qwen3-next", {"tp": 2}), ("tiny-deepseek", {"tp": 2}),
                                        ("tiny-deepseek-v4", {"pp": 3}), ("tiny-qwen3-moe", {"tp": 2}),
                                        ("tiny-minimax", {"tp": 2}), ("tiny-minimax", {"tp": 2, "sp": False}),
                                        ("tiny-deepseek-v4", {"tp": 2}), ("tiny-mimo", {"pp": 2})])
def test_newer_families_match_single_process(model, dims):
    """Hybrid linear attention under TP+SP, MLA + DSA under TP+SP, hyper-connection streams across pipeline stages."""
    ov = {"moe_aux_loss_coeff": 0.0} if model != "tiny-deepseek-v4" else {}
    world = dims.get("tp", 1) * dims.get("pp", 1)
    ref = _single(model, 2, ov)
    res = run_distributed(_run, world, model, dict(dims), 2, ov)
    pp = dims.get("pp", 1)
    _check(ref, res, lambda r: r // (world // pp) == pp - 1, tol=1e-3)


def _run_cp(rank, world, comm):
    from loongforge_b200.parallel import context_parallel as CP

    CP.set_cp_comm_type(comm)
    return _run(rank, world, "tiny-llama", {"cp": 2}, 3, {})


@pytest.mark.parametrize("comm", ["a2a", "allgather", "p2p"])
def test_context_parallel_matches_single_process(comm):
    ref = _single("tiny-llama", 3, {})
    res = run_distributed(_run_cp, 2, comm)
    _check(ref, res, lambda r: False)
    # the two cp ranks report the same (cp-summed, dp-averaged) loss
    for (l0, _), (l1, _) in zip(ref, res[0]):
        assert abs(l0 - l1) < 5e-4 * abs(l0), (l0, l1)


def _run_cp_two_level(rank, world):
    from loongforge_b200.parallel import context_parallel as CP
    from loongforge_b200.parallel import state as ps

    CP.set_cp_comm_type("a2a+p2p", 2)
    out = _run(rank, world, "tiny-llama", {"cp": 4}, 3, {})
    st = ps.get_state()
    assert CP._CFG["comm_type"] == "a2a+p2p"
    assert st.ranks("cp_inner") == [rank // 2 * 2, rank // 2 * 2 + 1] and st.ranks("cp_outer") == [rank % 2, rank % 2 + 2]
    return out


def test_two_level_context_parallel_matches_single_process():
    """cp = 4 as Ulysses inside pairs of neighbouring ranks and a KV ring between the pairs."""
    ref = _single("tiny-llama", 3, {})
    res = run_distributed(_run_cp_two_level, 4)
    for (l0, g0), (l1, g1) in zip(ref, res[0]):
        assert abs(l0 - l1) < 5e-4 * abs(l0) and abs(g0 - g1) < 5e-4 * max(1.0, abs(g0)), (ref, res[0])


def _run_cp_short_table(rank, world):
    return _run(rank, world, "tiny-llama", {"cp": 2}, 2, {"max_position_embeddings": 16})


def test_context_parallel_rows_longer_than_the_trained_context():
    """The rotary table must cover the positions of the whole row (cp x the rank's tokens), not only as many rows as the
    rank holds tokens: 64-token rows, 32 tokens per rank, a configured context of 16."""
    ref = _single("tiny-llama", 2, {"max_position_embeddings": 16})
    res = run_distributed(_run_cp_short_table, 2)
    for (l0, _), (l1, _) in zip(ref, res[0]):
        assert abs(l0 - l1) < 5e-4 * abs(l0), (l0, l1)


def test_sparse_attention_sequence_first_matches_single_process():
    """Sequence-first sparse attention under TP + SP: every rank attends from its own tokens with all heads against the
    gathered compressed keys (replicated up / output projections); same trajectory as one process, incl. the indexer
    loss and packed position handling."""
    ov = {"dsa_sp_first": True}
    ref = _single("tiny-deepseek", 3, {})
    res = run_distributed(_run, 2, "tiny-deepseek", {"tp": 2}, 3, ov)
    _check(ref, res, lambda r: True, tol=5e-4)
