"""Checkpoints written under one parallel layout must load under another (model weights), and resume exactly
under the same layout (weights + sharded optimizer state), including virtual pipeline chunks and the word
embedding that the first and last pipeline stage share."""
import tempfile

import pytest

from dist_utils import run_distributed

SEQ, GBS = 64, 4


def _trainer(model, dims_kw, ov):
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    dims_kw = dict(dims_kw)
    cfg = get_model_config(model, **ov)
    if dims_kw.get("tp", 1) > 1:
        cfg.sequence_parallel = True
    tc = TrainConfig(micro_batch_size=1, global_batch_size=GBS, seq_length=SEQ, train_iters=8, lr=1e-3, clip_grad=1.0,
                     log_interval=1000)
    return Trainer(cfg, tc, ParallelDims(**dims_kw)), cfg


def _iterator(tr, cfg, start=0):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator

    st = tr.st
    return synthetic_batch_iterator(cfg.vocab_size, SEQ, 1, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=5,
                                    pin_memory=False, start_sample=start)


def _save_worker(rank, world, tmp, model, dims_kw, ov, steps_before, steps_after):
    tr, cfg = _trainer(model, dims_kw, ov)
    it = _iterator(tr, cfg)
    for _ in range(steps_before):
        tr.train_step(it)
    tr.save_checkpoint(tmp)
    return [tr.train_step(it) for _ in range(steps_after)]


def _load_worker(rank, world, tmp, model, dims_kw, ov, steps_after):
    tr, cfg = _trainer(model, dims_kw, ov)
    assert tr.load_checkpoint(tmp) > 0
    it = _iterator(tr, cfg, start=tr.consumed_samples)
    return [tr.train_step(it) for _ in range(steps_after)]


def _losses(res):
    """Loss trajectory reported by whichever rank holds the last pipeline stage."""
    for out in res:
        if out and out[0].get("lm loss") is not None:
            return [m["lm loss"] for m in out], [m["grad_norm"] for m in out]
    raise AssertionError("no rank reported a loss")


@pytest.mark.parametrize("model,ov,save_dims,save_world,load_dims,load_world", [
    ("tiny-llama", {}, {"tp": 2}, 2, {"pp": 2}, 2),
    ("tiny-llama", {"num_layers": 4}, {"pp": 2, "vpp": 2}, 2, {"tp": 2}, 2),
    ("tiny-qwen3-moe", {"moe_aux_loss_coeff": 0.0}, {"ep": 2}, 2, {"tp": 2}, 2),
    ("tiny-minimax", {"untie_embeddings_and_output_weights": False}, {"pp": 2}, 2, {}, 1),
])
def test_weights_reshard_between_layouts(model, ov, save_dims, save_world, load_dims, load_world):
    with tempfile.TemporaryDirectory() as tmp:
        a = run_distributed(_save_worker, save_world, tmp, model, save_dims, ov, 2, 1)
        b = run_distributed(_load_worker, load_world, tmp, model, load_dims, ov, 1)
    (la, ga), (lb, gb) = _losses(a), _losses(b)
    # the first step after loading sees exactly the saved weights: same loss and same gradient norm
    assert abs(la[0] - lb[0]) < 1e-3 * max(1.0, abs(la[0])), (la, lb)
    assert abs(ga[0] - gb[0]) < 5e-3 * max(1.0, abs(ga[0])), (ga, gb)


@pytest.mark.parametrize("model,ov,dims,world", [
    ("tiny-llama", {"num_layers": 4}, {"pp": 2, "vpp": 2}, 2),
    ("tiny-minimax", {"untie_embeddings_and_output_weights": False}, {"pp": 2}, 4),
])
def test_resume_continues_the_trajectory(model, ov, dims, world):
    """Same layout: weights and optimizer moments come back, so two further steps match the uninterrupted run."""
    with tempfile.TemporaryDirectory() as tmp:
        a = run_distributed(_save_worker, world, tmp, model, dims, ov, 2, 2)
        b = run_distributed(_load_worker, world, tmp, model, dims, ov, 2)
    (la, ga), (lb, gb) = _losses(a), _losses(b)
    for x, y in zip(la + ga, lb + gb):
        assert abs(x - y) < 1e-5 * max(1.0, abs(x)), (la, lb, ga, gb)
