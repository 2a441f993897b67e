"""CLI parsing, YAML composition (defaults lists, resolvers, overrides) and validation."""
import os
import textwrap

import pytest


def test_yaml_compose_defaults_resolvers_overrides(tmp_path, monkeypatch):
    from loongforge_b200.config import yaml_compose as yc

    (tmp_path / "enc").mkdir()
    (tmp_path / "enc" / "vit.yaml").write_text("hidden_size: 64\nactivation_func: ${act:silu}\n")
    (tmp_path / "lm.yaml").write_text("num_layers: 2\nfreq: ${moe_freq:[0]*1+[1]*3}\n")
    (tmp_path / "top.yaml").write_text(textwrap.dedent("""
        defaults:
          - enc@model.image_encoder: vit
          - .@model.foundation: lm
          - _self_
        model:
          root: ${oc.env:MY_ROOT,/x}/cfg
          foundation:
            num_layers: 4
          ref: ${model.foundation.num_layers}
    """))
    monkeypatch.delenv("MY_ROOT", raising=False)
    cfg = yc.compose(str(tmp_path / "top.yaml"), ["model.foundation.num_layers=6", "+model.image_encoder.freeze=true",
                                                  "~model.image_encoder.activation_func"])
    assert cfg["model"]["foundation"]["num_layers"] == 6 and cfg["model"]["ref"] == 6
    assert cfg["model"]["foundation"]["freq"] == [0, 1, 1, 1]
    assert cfg["model"]["image_encoder"] == {"hidden_size": 64, "freeze": True}
    assert cfg["model"]["root"] == "/x/cfg"
    with pytest.raises(KeyError):
        yc.compose(str(tmp_path / "top.yaml"), ["model.nope=1"])


def test_cli_to_configs(monkeypatch):
    from loongforge_b200.config.arguments import parse_args
    from loongforge_b200.config.build import build_configs

    monkeypatch.setenv("WORLD_SIZE", "8")
    args, ov = parse_args(["--model-name", "llama3-8b", "--tensor-model-parallel-size", "2", "--sequence-parallel",
                           "--tp-comm-overlap", "--use-distributed-optimizer", "--seq-length", "8192",
                           "--micro-batch-size", "1", "--global-batch-size", "128", "--bf16", "--train-iters", "10"])
    cfg, tc, dims, _ = build_configs(args, ov)
    assert (cfg.num_layers, cfg.hidden_size, cfg.num_query_groups, cfg.ffn_hidden_size) == (32, 4096, 8, 14336)
    assert cfg.sequence_parallel and cfg.tp_comm_overlap and dims.tp == 2 and tc.global_batch_size == 128
    with pytest.raises(SystemExit):
        parse_args(["--model-name", "llama3-8b", "--no-such-flag"])
    args, ov = parse_args(["--model-name", "llama3-8b", "--global-batch-size", "3", "--seq-length", "128"])
    with pytest.raises(ValueError):
        build_configs(args, ov)


def test_registry_presets_cover_baseline_configs():
    from loongforge_b200.models.registry import get_model_config

    q = get_model_config("qwen3-30b-a3b")
    assert (q.num_moe_experts, q.moe_router_topk, q.moe_ffn_hidden_size, q.qk_layernorm) == (128, 8, 768, True)
    d = get_model_config("deepseek-v3.2-slice")
    assert d.use_dsa and d.num_layers == 4 and d.moe_layer_freq == [0, 1, 1, 1] and d.fp8 == "blockwise"
    n = get_model_config("llama3-8b").num_parameters()
    assert 7.9e9 < n < 8.2e9


def test_every_model_yaml_builds_the_registered_preset():
    """The YAML files under configs/models and the registry presets describe the same models."""
    import dataclasses
    from loongforge_b200.config import build as B
    from loongforge_b200.config import yaml_compose
    from loongforge_b200.models.registry import get_model_config, list_models

    checked = 0
    for name, rel in B.MODEL_YAML.items():
        if name not in list_models() or name in ("llama3-8b", "qwen2.5-7b", "qwen3-30b-a3b", "deepseek-v3.2"):
            continue  # the hand-written files use the reference's key spelling and are covered above
        raw = yaml_compose.compose(os.path.join(B.CONFIG_DIR, rel))
        cfg = B.transformer_config_from_yaml({k: v for k, v in raw.items() if not isinstance(v, dict)})
        ref = get_model_config(name)
        for f in dataclasses.fields(cfg):
            if f.name in ("params_dtype", "padded_vocab_size", "output_layer_init_std", "model_family"):
                continue
            assert getattr(cfg, f.name) == getattr(ref, f.name), (name, f.name)
        checked += 1
    assert checked >= 20



def test_reference_flags_and_entry_point_are_accepted():
    """Every flag the reference defines itself (147) parses, the `loongforge.train` entry objects exist, and the
    freezing flags reach the trainer."""
    import re

    from loongforge_b200.config.arguments import build_parser, parse_args

    known = {o for a in build_parser()._actions for o in a.option_strings}
    for f in ("--loss-reduction", "--freeze-parameters-regex", "--log-tensor-stage", "--dp-balance-verbose",
              "--hf-dequantize-int4", "--max-latent-height", "--energon-pack-algo", "--initial-loss-scale"):
        assert f in known, f
    args, _ = parse_args(["--model-name", "tiny-llama", "--freeze-parameters", "embedding", "output_layer",
                          "--freeze-parameters-regex", r"layers\\.0\\.", "--force_pow_2_scales", "--enable-ema"])
    assert args.freeze_parameters == ["embedding", "output_layer"] and args.force_pow_2_scales and args.enable_ema
    assert re.compile(args.freeze_parameters_regex)
    import loongforge.train as entry

    assert callable(entry.main) and callable(entry.parse_train_args) and callable(entry.build_model_trainer)


def test_freeze_parameters_flags_freeze_before_the_optimizer_is_built():
    import torch

    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=2, ffn_hidden_size=128, vocab_size=128)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=16, train_iters=1,
                     freeze_parameters=["embedding"], freeze_parameters_regex=r"layers\.0\.")
    tr = Trainer(cfg, tc, device=torch.device("cpu"))
    named = dict(tr.models[0].module.named_parameters())
    frozen = [n for n, p in named.items() if not p.requires_grad]
    assert frozen and all(n.startswith("embedding") or "layers.0." in n for n in frozen)
    assert any("layers.1." in n and p.requires_grad for n, p in named.items())
    from loongforge_b200.data.synthetic import synthetic_batch_iterator

    before = {n: p.detach().clone() for n, p in named.items()}
    tr.train_step(synthetic_batch_iterator(128, 16, 1))
    for n, p in named.items():
        changed = not torch.equal(before[n], p.detach())
        assert changed == p.requires_grad or not p.requires_grad and not changed, n


def test_validator_rule_families():
    """SFT, MoE, overlap-schedule and multimodal rules raise on inconsistent flags and fix up derived ones."""
    import types

    import pytest

    from loongforge_b200.config import validators as V
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig

    def ns(**kw):
        return types.SimpleNamespace(**kw)

    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=64, training_phase="sft")
    with pytest.raises(ValueError, match="packs one row"):
        V._validate_sft(ns(packing_sft_data=True), tc)
    with pytest.raises(ValueError, match="cannot both"):
        V._validate_sft(ns(train_on_prompt=True, history_mask_loss=True), tc)
    with pytest.raises(KeyError):
        V._validate_sft(ns(chat_template="no_such_template"), TrainConfig(training_phase="sft"))
    V._validate_sft(ns(chat_template="qwen3_hf_training"), TrainConfig(training_phase="sft"))

    moe = get_model_config("tiny-qwen3-moe")
    dense = get_model_config("tiny-llama")
    over = TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=64, overlap_moe_expert_parallel_comm=True)
    with pytest.raises(ValueError, match="at least two"):
        V._validate_attention_variants(ns(), moe, over, ParallelDims())
    over.global_batch_size = 4
    V._validate_attention_variants(ns(), moe, over, ParallelDims())
    with pytest.raises(ValueError, match="MoE model"):
        V._validate_attention_variants(ns(), dense, over, ParallelDims())
    with pytest.raises(ValueError, match="pipeline size 1"):
        V._validate_attention_variants(ns(), moe, over, ParallelDims(pp=2))

    a = ns(moe_token_dispatcher_type="allgather")
    V._validate_moe(a, dense, tc, ParallelDims())
    assert a.moe_token_dispatcher_type == "alltoall"
    bad = get_model_config("tiny-qwen3-moe", moe_router_topk=9)
    with pytest.raises(ValueError, match="exceeds"):
        V._validate_moe(ns(), bad, tc, ParallelDims())
    grp = get_model_config("tiny-qwen3-moe", moe_router_num_groups=4, moe_router_group_topk=1, moe_router_topk=3)
    with pytest.raises(ValueError, match="cannot hold"):
        V._validate_moe(ns(), grp, tc, ParallelDims())

    a = ns(max_text_length=510, encoder_tensor_model_parallel_size=1, model_name="wan2-1-i2v", num_frames=81, height=480, width=832)
    V._validate_multimodal(a, dense, tc, ParallelDims(cp=4))
    assert a.max_text_length == 512
    with pytest.raises(ValueError, match="4 k \\+ 1"):
        V._validate_multimodal(ns(model_name="wan2-1-i2v", num_frames=80), dense, tc, ParallelDims())
    with pytest.raises(ValueError, match="divide by the encoder"):
        V._validate_multimodal(ns(encoder_tensor_model_parallel_size=3), dense, tc, ParallelDims(tp=4))


def test_flags_of_the_reference_training_launchers_are_all_accepted():
    """Every ``--flag`` that a training launcher of the reference passes to its entry point is an option of this
    parser (the launchers are read as text; skipped when no reference tree sits beside the repository)."""
    import glob
    import os
    import re

    import pytest

    from loongforge_b200.config.arguments import build_parser

    ref = os.environ.get("LOONGFORGE_REFERENCE_DIR") or os.path.join(os.path.dirname(__file__), "..", "..", "reference")
    scripts = [f for f in glob.glob(os.path.join(ref, "examples", "**", "*.sh"), recursive=True)
               if "loongforge/train.py" in open(f, errors="ignore").read()]
    if not scripts:
        pytest.skip("no reference tree beside the repository")
    known = {o for a in build_parser()._actions for o in a.option_strings}
    not_ours = {"--nproc_per_node", "--nnodes", "--node_rank", "--master_addr", "--master_port", "--rdzv_backend",
                "--rdzv_endpoint", "--rdzv_id", "--max_restarts",
                # flags of the profiler some launchers wrap the command in
                "--version", "--force-overwrite", "--capture-range", "--capture-range-end"}
    unknown = {}
    for f in scripts:
        text = "\n".join(l for l in open(f, errors="ignore").read().splitlines() if not l.strip().startswith("#"))
        for m in re.finditer(r"(?<![\w-])(--[a-z][a-z0-9_-]+)", text):
            flag = m.group(1)
            if flag in not_ours or flag in known or flag.replace("_", "-") in known:
                continue
            unknown.setdefault(flag, []).append(os.path.relpath(f, ref))
    assert len(scripts) > 100 and not unknown, {k: v[:2] for k, v in unknown.items()}


def test_model_yamls_of_the_reference_compose_unchanged(monkeypatch):
    """The reference's own ``configs/models/**/*.yaml`` (Hydra ``_target_`` keys, defaults lists, custom resolvers) go
    through this composer and the model-config builder as they are (skipped without a reference tree)."""
    import glob
    import os

    import pytest

    from loongforge_b200.config import yaml_compose as Y
    from loongforge_b200.config.build import transformer_config_from_yaml

    ref = os.environ.get("LOONGFORGE_REFERENCE_DIR") or os.path.join(os.path.dirname(__file__), "..", "..", "reference")
    files = [f for f in glob.glob(os.path.join(ref, "configs", "models", "**", "*.yaml"), recursive=True)
             if "ckpt_convert" not in f]
    if not files:
        pytest.skip("no reference tree beside the repository")
    monkeypatch.setenv("LOONGFORGE_PATH", os.path.abspath(ref))
    built = {}
    for f in files:
        try:
            raw = Y.compose(f)
        except KeyError as e:
            if "environment variable" in str(e):
                continue  # embodied recipes interpolate checkpoint locations from the environment
            raise
        node = raw.get("model", raw)
        node = node["foundation"] if isinstance(node, dict) and "foundation" in node else node
        built[os.path.relpath(f, ref)] = transformer_config_from_yaml({k: v for k, v in node.items() if not isinstance(v, dict)})
    assert len(built) > 100
    ll = built[os.path.join("configs", "models", "llama3", "llama3_8b.yaml")]
    assert (ll.num_layers, ll.hidden_size, ll.ffn_hidden_size, ll.num_query_groups) == (32, 4096, 14336, 8)
    assert ll.gated_linear_unit and ll.model_family == "llama"
