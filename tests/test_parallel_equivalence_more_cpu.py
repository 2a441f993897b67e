"""More layouts against the single-process trajectory: interleaved pipeline, shared embeddings across stages, context
parallelism with several rows per micro-batch, newer model families (second part of test_parallel_equivalence_cpu.py,
split so that test workers can run the two halves side by side)."""
import pytest

from dist_utils import run_distributed
from test_parallel_equivalence_cpu import _check, _run, _single


@pytest.mark.parametrize("model,dims,ov,world", [
    ("tiny-llama", {"pp": 2, "vpp": 2}, {"num_layers": 4}, 2),          # interleaved 1F1B
    ("tiny-deepseek", {"cp": 2}, {"moe_aux_loss_coeff": 0.0}, 2),       # MLA + DSA with context parallel keys
    ("tiny-qwen3-moe", {"tp": 2, "ep": 2}, {"moe_aux_loss_coeff": 0.0}, 4),
    ("tiny-minimax", {"pp": 2}, {}, 2),                                  # MoE + MTP on the last pipeline stage
    ("tiny-qwen3-moe", {"tp": 2}, {"moe_z_loss_coeff": 1e-3}, 2),        # aux + z loss over sequence shards
    ("tiny-qwen3-moe", {"tp": 2, "sp": False}, {"moe_z_loss_coeff": 1e-3}, 2),   # MoE shards its tokens itself
    ("tiny-llama", {"pp": 2}, {"untie_embeddings_and_output_weights": False}, 2),   # tied embedding across stages
    ("tiny-minimax", {"pp": 2}, {"untie_embeddings_and_output_weights": False}, 4),  # + sharded optimizer over dp 2
])
def test_more_layouts_match_single_process(model, dims, ov, world):
    ref = _single(model, 2, ov)
    res = run_distributed(_run, world, model, dict(dims), 2, ov)
    pp = dims.get("pp", 1)
    _check(ref, res, lambda r: r // (world // pp) == pp - 1, tol=1e-3)


@pytest.mark.parametrize("model,dims,ov,world", [
    ("tiny-minimax", {"cp": 2}, {}, 2),                      # MTP shifts across context-parallel chunk boundaries
    ("tiny-deepseek", {"cp": 2}, {"use_dsa": False}, 2),     # dense MLA through ring attention
    ("tiny-llama", {"tp": 2, "cp": 2}, {}, 4),
    ("tiny-ernie-vl", {"tp": 2}, {}, 2),                     # shared expert over the gathered sequence
    ("tiny-qwen3-next", {"cp": 2}, {"moe_aux_loss_coeff": 0.0}, 2),   # convolution + delta rule on the gathered sequence
    ("tiny-deepseek-v4", {"cp": 2, "tp": 2}, {}, 4),         # compressed sparse attention on the gathered sequence
])
def test_two_rows_per_microbatch_match_single_process(model, dims, ov, world):
    """Micro-batches of two rows: context parallelism slices every row separately."""
    ref = _single(model, 2, ov, mbs=2)
    res = run_distributed(_run, world, model, dict(dims), 2, ov, 4, 2)
    _check(ref, res, lambda r: True, tol=1e-3)


@pytest.mark.parametrize("model,dims,ov,world,gbs", [
    ("tiny-llama", {"pp": 2, "vpp": 2}, {"num_layers": 4}, 2, 8),      # two groups of micro-batches in one stream
    ("tiny-llama", {"pp": 3, "vpp": 2}, {"num_layers": 6}, 3, 6),
    ("tiny-minimax", {"pp": 2, "vpp": 2}, {"num_layers": 4, "untie_embeddings_and_output_weights": False}, 2, 4),
])
def test_interleaved_schedule_matches_single_process(model, dims, ov, world, gbs):
    ref = _single(model, 2, ov, gbs)
    res = run_distributed(_run, world, model, dict(dims), 2, ov, gbs)
    _check(ref, res, lambda r: r == world - 1, tol=1e-3)
