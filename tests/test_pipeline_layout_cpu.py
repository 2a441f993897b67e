"""Pipeline layout strings, custom per-stage layer counts, and an uneven pipeline that must train like one process."""
import pytest

from loongforge_b200.parallel import pipeline_layout as PLY


def test_layout_string_expansion_and_counts():
    assert PLY.expand_layout("Et*3|(tt|)*2,m,L") == ["Ettt", "tt", "tt", "mL"]
    assert PLY.expand_layout("E t | (t|)*2 t L") == ["Et", "t", "t", "tL"]
    assert PLY.layers_per_virtual_stage("Et*3|(tt|)*2,m,L", pp=4, num_layers=7, mtp_num_layers=1) == [3, 2, 2, 0]
    # pp 2 x 2 virtual stages: chunk 0 of both ranks, then chunk 1 of both ranks
    assert PLY.layers_per_virtual_stage("Ett|t|tt|tL", pp=2, vpp=2, num_layers=6) == [2, 1, 2, 1]
    assert PLY.layout_from_counts([2, 1, 2, 1], mtp_num_layers=1) == "Ett|t|tt|tmL"


@pytest.mark.parametrize("layout,err", [
    ("Ett|tt", ValueError),            # no loss stage
    ("tt|EtL", ValueError),            # embedding not first
    ("Ett|ttL|t", ValueError),         # loss not last
    ("Et|m|L", NotImplementedError),   # MTP away from the loss stage
    ("Et|t(L", ValueError),
    ("Ex|tL", ValueError),
])
def test_layout_errors(layout, err):
    with pytest.raises(err):
        PLY.layers_per_virtual_stage(layout, pp=len(layout.split("|")), mtp_num_layers=1)


def test_custom_layer_spellings():
    assert PLY.split_rank_layers_over_virtual_stages([5, 4], 2) == [2, 2, 3, 2]
    assert PLY.resolve_stage_layers(9, 2, 2, custom_pipeline_layers=[5, 4]) == [2, 2, 3, 2]
    assert PLY.resolve_stage_layers(9, 2, 2, custom_virtual_pipeline_layers=[1, 2, 3, 3]) == [1, 2, 3, 3]
    assert PLY.resolve_stage_layers(8, 2) is None
    with pytest.raises(ValueError):
        PLY.resolve_stage_layers(8, 2, custom_pipeline_layers=[5, 4])
    with pytest.raises(ValueError):
        PLY.resolve_stage_layers(9, 2, layout="Ettttt|ttttL", custom_pipeline_layers=[5, 4])


def test_cli_layout_reaches_the_train_config(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "2")
    from loongforge_b200.config.arguments import parse_args
    from loongforge_b200.config.build import build_configs

    args, ov = parse_args(["--model-name", "tiny-llama", "--num-layers", "4", "--pipeline-model-parallel-size", "2",
                       "--pipeline-model-parallel-layout", "Et|tttL", "--custom-pipeline-recompute-layers", "1,0",
                       "--micro-batch-size", "1", "--global-batch-size", "2", "--seq-length", "64",
                       "--train-iters", "1", "--mock-data"])
    cfg, tc, dims = build_configs(args, ov)[:3]
    assert tc.custom_pipeline_layers == [1, 3] and tc.custom_pipeline_recompute_layers == [1, 0]


def _uneven(rank, world, custom, recompute):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-llama", num_layers=4)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=2, lr=1e-3, clip_grad=1.0,
                     log_interval=1000, custom_pipeline_layers=custom, custom_pipeline_recompute_layers=recompute)
    tr = Trainer(cfg, tc, ParallelDims(pp=world))
    if custom:
        assert len(tr.models[0].module.decoder.layers) == custom[tr.st.pp_rank]
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, seed=3, pin_memory=False)
    return [(m.get("lm loss"), m["grad_norm"]) for m in (tr.train_step(it) for _ in range(2))]


def test_uneven_pipeline_with_per_stage_recompute_matches_one_process():
    from dist_utils import run_distributed

    ref = run_distributed(_uneven, 1, None, None)[0]
    res = run_distributed(_uneven, 2, [1, 3], [1, 2])
    for (l0, g0), (l1, g1) in zip(ref, res[1]):
        assert abs(l0 - l1) < 2e-4 * abs(l0) and abs(g0 - g1) < 5e-3 * max(1, g0), (ref, res)
