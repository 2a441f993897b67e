"""Hidden / attention dropout with the tensor-parallel-aware random streams: masks agree where activations are
replicated over the TP group and differ where they are sharded, recomputation replays them, and a checkpoint carries
the tracked streams so that a resumed run draws the same masks."""
import os

import torch

from dist_utils import run_distributed


def _trainer(ov=None, tc_ov=None, dims=None):
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    kw = dict(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, vocab_size=512,
              hidden_dropout=0.2, attention_dropout=0.1)
    kw.update(ov or {})
    cfg = TransformerConfig(**kw)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=32, train_iters=4, lr=1e-3, seed=11,
                     **(tc_ov or {}))
    return Trainer(cfg, tc, ParallelDims(**(dims or {})), device=torch.device("cpu"))


def _losses(tr, n, seed=5):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator

    it = synthetic_batch_iterator(512, 32, 1, dp_rank=tr.st.dp_rank, dp_size=tr.st.dp_size, seed=seed)
    return [tr.train_step(it)["lm loss"] for _ in range(n)]


def test_dropout_changes_training_but_not_evaluation_and_recompute_replays_it():
    a = _losses(_trainer(), 3)
    b = _losses(_trainer(), 3)
    assert a == b  # same seed, same masks
    c = _losses(_trainer({"hidden_dropout": 0.0, "attention_dropout": 0.0}), 3)
    assert a != c
    # full recomputation draws the same masks in the replay: identical trajectory
    r = _losses(_trainer({"recompute_granularity": "full", "recompute_method": "uniform", "recompute_num_layers": 1}), 3)
    assert max(abs(x - y) for x, y in zip(a, r)) < 1e-6, (a, r)


def _tp_worker(rank, world, sp):
    tr = _trainer({"sequence_parallel": sp}, dims={"tp": 2})
    losses = _losses(tr, 2)
    from loongforge_b200.parallel.random import MODEL_PARALLEL_RNG, get_rng_tracker

    return losses, get_rng_tracker().get_states()[MODEL_PARALLEL_RNG].sum().item(), torch.get_rng_state().sum().item()


def test_tp_ranks_share_the_default_stream_and_differ_in_the_tracked_one():
    for sp in (False, True):
        (l0, t0, d0), (l1, t1, d1) = run_distributed(_tp_worker, 2, sp)
        assert l0 == l1 and all(x == x for x in l0)   # one loss for the TP group, finite
        assert d0 == d1                               # default stream stays in lock step over the TP group
        assert t0 != t1                               # model-parallel stream differs per TP rank


def test_checkpoint_carries_the_tracked_streams(tmp_path):
    tr = _trainer(tc_ov={"save": str(tmp_path)})
    _losses(tr, 2)
    tr.save_checkpoint(str(tmp_path))
    from loongforge_b200.data.synthetic import synthetic_batch_iterator

    it = synthetic_batch_iterator(512, 32, 1, seed=9)
    nxt = tr.train_step(it)["lm loss"]
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    tr2 = _trainer(tc_ov={"load": str(tmp_path)})
    tr2.load_checkpoint(str(tmp_path))
    it2 = synthetic_batch_iterator(512, 32, 1, seed=9)
    assert tr2.train_step(it2)["lm loss"] == nxt
