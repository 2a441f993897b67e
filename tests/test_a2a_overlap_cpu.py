"""The MoE all-to-all overlap schedule (forward of micro-batch i issued node by node between the backward nodes of
micro-batch i - 1) must reproduce the plain step: same losses and gradient norms over several optimizer steps, on one
process and with expert / tensor parallelism on gloo ranks."""
import pytest
import torch

from dist_utils import run_distributed


def _run(rank, world, model_name, dims_kw, overlap, overrides, steps=3, gbs=4):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config(model_name, **overrides)
    if dims_kw.get("tp", 1) > 1:
        cfg.sequence_parallel = dims_kw.pop("sp", True)
    dims_kw.pop("sp", None)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=gbs, seq_length=64, train_iters=steps, lr=1e-3,
                     clip_grad=1.0, log_interval=1000, overlap_moe_expert_parallel_comm=overlap)
    tr = Trainer(cfg, tc, ParallelDims(**dims_kw))
    st = tr.st
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=3,
                                  pin_memory=False)
    out = []
    for _ in range(steps):
        m = tr.train_step(it)
        out.append((m["lm loss"], m["grad_norm"]))
    trace = list(tr._a2a_executor.trace) if overlap else []
    return out, trace


def _same(a, b, tol=1e-5):
    for (l0, g0), (l1, g1) in zip(a, b):
        assert abs(l0 - l1) <= tol * max(1.0, abs(l0)), (l0, l1)
        assert abs(g0 - g1) <= tol * max(1.0, abs(g0)), (g0, g1)


@pytest.mark.parametrize("model,ov", [("tiny-qwen3-moe", {}), ("tiny-deepseek", {}),
                                      ("tiny-qwen3-moe", {"hidden_dropout": 0.1})])
def test_overlap_schedule_matches_plain_step_single_process(model, ov):
    plain, _ = run_distributed(_run, 1, model, {}, False, ov)[0]
    over, trace = run_distributed(_run, 1, model, {}, True, ov)[0]
    _same(plain, over)
    # micro-batch 1's forward nodes are issued between micro-batch 0's backward nodes, exchange before compute
    i = trace.index("bwd0.L1.combine") if "bwd0.L1.combine" in trace else trace.index("bwd0.L0.combine")
    assert trace[i + 1].startswith("fwd1."), trace[i - 2:i + 3]
    assert any(t.startswith("fwd1.") and t.endswith(".dispatch") for t in trace)


@pytest.mark.parametrize("dims", [{"ep": 2}, {"tp": 2, "ep": 2}, {"tp": 2, "etp": 2}, {"tp": 2, "sp": False}])
def test_overlap_schedule_matches_plain_step_parallel(dims):
    ov = {"moe_aux_loss_coeff": 1e-2}
    world = 2
    plain = run_distributed(_run, world, "tiny-qwen3-moe", dict(dims), False, ov)
    over = run_distributed(_run, world, "tiny-qwen3-moe", dict(dims), True, ov)
    for (p, _), (o, _) in zip(plain, over):
        _same(p, o)


def test_segment_gradients_sum_where_a_value_feeds_two_nodes():
    from loongforge_b200.runtime import a2a_overlap as A

    w = torch.nn.Parameter(torch.tensor([2.0, 3.0]))
    segs = [A.Segment("a", A.COMPUTE, [], ["x"], lambda: w * 1.0),
            A.Segment("b", A.COMM, ["x"], ["y"], lambda x: x * x),
            A.Segment("c", A.COMPUTE, ["x", "y"], ["loss"], lambda x, y: (x + y).sum())]
    prog = A.MicrobatchProgram(segs, 0)
    A._seed_loss_gradient(prog)
    A.run_overlapped([prog])
    assert torch.allclose(w.grad, 1 + 2 * w.detach())  # d/dw (w + w^2)
