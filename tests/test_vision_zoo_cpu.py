"""Vision encoder families and projectors: shapes, gradient flow, and the distinctive option of each."""
import pytest
import torch

from loongforge_b200.models.config import TransformerConfig
from loongforge_b200.models import vision_zoo as VZ
from loongforge_b200.parallel import state as ps


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=64, num_attention_heads=4, kv_channels=16, ffn_hidden_size=128, vocab_size=0,
                normalization="LayerNorm", activation="gelu", gated_linear_unit=False, add_bias_linear=True,
                add_qkv_bias=True, layernorm_epsilon=1e-6, causal=False, patch_size=14, temporal_patch_size=1,
                spatial_merge_size=2, position_embedding_type="rope")
    base.update(kw)
    return TransformerConfig(**base)


@pytest.fixture(autouse=True)
def _state():
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    yield


GRID = torch.tensor([[1, 4, 6], [2, 2, 4]])
N_PATCH = 1 * 4 * 6 + 2 * 2 * 4


def _pixels(cfg):
    return torch.randn(N_PATCH, cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size ** 2)


@pytest.mark.parametrize("family", sorted(VZ.VISION_FAMILIES))
def test_family_forward_backward(family):
    cfg = _cfg(qk_layernorm_full=(family == "intern_vit"))
    torch.manual_seed(0)
    opts, adapter_cls = VZ.VISION_FAMILIES[family]
    over = {"deepstack_indexes": (0, 1)} if family == "qwen3_vl_vit" else {}
    if opts.get("pos_table_side"):
        over["pos_table_side"] = 8
    vit = VZ.build_vision_encoder(family, cfg, **over)
    x, taps = vit(_pixels(cfg), GRID)
    n_tok = N_PATCH + (3 if family == "intern_vit" else 0)  # one class token per frame
    assert x.shape == (n_tok, 64)
    out = x
    if adapter_cls is not None:
        ad = adapter_cls(cfg, 96)
        out = ad(x, GRID)
        units = 1 * 2 * 3 + 2 * 1 * 2
        expect = units if family != "ernie_vit" else 1 * 2 * 3 + 1 * 1 * 2  # temporal fold of 2 (single frame repeated)
        assert out.shape == (expect, 96), out.shape
    if family == "qwen3_vl_vit":
        assert len(taps) == 2
        feats = VZ.DeepStackMergers(cfg, 96, 2)(taps, GRID)
        assert all(f.shape == (10, 96) for f in feats)
        out = out.sum() + sum(f.sum() for f in feats)
    out.sum().backward()
    assert all(p.grad is not None for p in vit.parameters())


def test_interpolated_position_table_matches_table_at_native_size():
    table = torch.randn(16, 8)
    e = VZ.interpolate_pos_table(table, 4, torch.tensor([[2, 4, 4]]))
    assert torch.allclose(e[:16], table, atol=1e-6) and torch.allclose(e[16:], table, atol=1e-6)


def test_layer_scale_zero_is_identity():
    cfg = _cfg()
    layer = VZ.LayerScaleLayer(cfg, 0, init_scale=0.0)
    x = torch.randn(10, 64)
    packed = VZ.PackedSeqParams(torch.tensor([0, 10], dtype=torch.int32), 10)
    assert torch.equal(layer(x, None, packed), x)


def test_deepstack_hook_adds_only_at_image_tokens():
    hidden = torch.zeros(6, 4)
    mask = torch.tensor([False, True, True, False, False, True])
    hook = VZ.make_deepstack_hook([torch.ones(3, 4), 2 * torch.ones(3, 4)], mask)
    assert hook(0, hidden)[mask].eq(1).all() and hook(0, hidden)[~mask].eq(0).all()
    assert hook(1, hidden)[mask].eq(2).all() and torch.equal(hook(2, hidden), hidden)


@pytest.mark.parametrize("family", ["qwen3_vl_vit", "intern_vit", "moon_vit"])
def test_omni_model_with_zoo_encoders(family):
    """Composed VLM: image tokens replaced by projected features (+ DeepStack taps added in the first LLM layers)."""
    from loongforge_b200.models.omni import OmniCombinationModel
    from loongforge_b200.models.registry import get_model_config

    lm = get_model_config("tiny-llama", vocab_size=300, num_layers=3)
    vit = _cfg(qk_layernorm_full=(family == "intern_vit"))
    over = {"pos_table_side": 8}
    if family == "qwen3_vl_vit":
        over["deepstack_indexes"] = (0, 1)
    torch.manual_seed(0)
    m = OmniCombinationModel(lm, vit, image_token_id=299, vision_family=family, vision_options=over)
    n_img_tok = 1 * 2 * 3 + 2 * 1 * 2
    tokens = torch.cat([torch.randint(0, 298, (5,)), torch.full((n_img_tok,), 299), torch.randint(0, 298, (7,))])
    T = tokens.numel()
    loss = m(tokens, torch.arange(T), pixels=_pixels(vit), grid_thw=GRID, labels=torch.roll(tokens, -1),
             loss_mask=torch.ones(T)).mean()
    loss.backward()
    assert torch.isfinite(loss)
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert not missing, missing
    if family == "qwen3_vl_vit":
        assert m.decoder.deepstack_hook is not None


def test_vlm_cli_with_internvit_yaml(tmp_path):
    """A composed VLM YAML whose encoder section names a zoo family trains through the CLI."""
    import subprocess
    import sys
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    y = tmp_path / "tiny_internvl.yaml"
    y.write_text("""
model:
  model_type: internvl
  image_encoder:
    model_type: intern_vit
    num_layers: 2
    hidden_size: 64
    kv_channels: 16
    ffn_hidden_size: 128
    num_attention_heads: 4
    num_query_groups: 4
    patch_size: 14
    temporal_patch_size: 1
    spatial_merge_size: 2
    normalization: LayerNorm
    activation: gelu
    gated_linear_unit: false
    add_bias_linear: true
    add_qkv_bias: true
    causal: false
    vocab_size: 0
    qk_layernorm_full: true
    vision_options: {pos_table_side: 4}
  foundation:
    model_type: llama
    num_layers: 2
    hidden_size: 64
    num_attention_heads: 4
    num_query_groups: 2
    ffn_hidden_size: 128
    vocab_size: 512
""")
    cmd = [sys.executable, "-m", "loongforge_b200.train", "--config-file", str(y), "--seq-length", "64",
           "--micro-batch-size", "1", "--global-batch-size", "2", "--train-iters", "3", "--lr", "1e-3",
           "--image-resolution", "56", "--log-interval", "1"]
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "iteration        3/" in p.stdout and "lm loss" in p.stdout


def test_vlm_cli_trains_from_image_text_shards(tmp_path):
    """Image-text records -> WebDataset shards (tool) -> reader -> task encoder -> online packer -> VLM trainer."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from loongforge_b200.data import multimodal as MM
    from tools.data_preprocess.vlm_to_webdataset import write_shards

    rng = np.random.RandomState(0)
    img_dir = tmp_path / "img"
    img_dir.mkdir()
    recs = []
    for i in range(12):
        np.save(img_dir / f"{i}.npy", rng.randint(0, 255, size=(56 + 28 * (i % 2), 56, 3), dtype=np.uint8))
        recs.append({"image": f"{i}.npy", "conversations": [{"from": "human", "value": "<image>what is shown?"},
                                                            {"from": "gpt", "value": "answer number %d" % i}]})
    idx = write_shards(recs, str(tmp_path / "wds"), image_root=str(img_dir), samples_per_shard=5)
    assert idx["total"] == 12 and len(idx["shards"]) == 3
    # the reader splits the stream over data-parallel ranks without overlap
    a = list(MM.webdataset_samples(str(tmp_path / "wds"), dp_rank=0, dp_size=2, epochs=1))
    b = list(MM.webdataset_samples(str(tmp_path / "wds"), dp_rank=1, dp_size=2, epochs=1))
    assert len(a) == len(b) == 6 and a[0]["images"][0].shape[2] == 3 and a[0]["conversation"][1]["role"] == "assistant"
    y = tmp_path / "tiny_vl.yaml"
    y.write_text(json.dumps({"model": {
        "model_type": "qwen2_5_vl",
        "image_encoder": {"model_type": "qwen2_5_vit", "num_layers": 2, "hidden_size": 64, "kv_channels": 16,
                          "ffn_hidden_size": 128, "num_attention_heads": 4, "num_query_groups": 4, "patch_size": 14,
                          "temporal_patch_size": 2, "spatial_merge_size": 2, "causal": False, "vocab_size": 0,
                          "fullatt_block_indexes": [1], "vision_window_size": 56},
        "foundation": {"model_type": "qwen2", "num_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
                       "num_query_groups": 2, "ffn_hidden_size": 128, "vocab_size": 512,
                       "position_embedding_type": "mrope", "mrope_section": [2, 3, 3]}}}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "loongforge_b200.train", "--config-file", str(y), "--seq-length", "128",
           "--micro-batch-size", "1", "--global-batch-size", "2", "--train-iters", "3", "--lr", "1e-3",
           "--log-interval", "1", "--data-path", str(tmp_path / "wds"), "--training-phase", "sft", "--mock-data"]
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "iteration        3/" in p.stdout and "lm loss" in p.stdout


def _vlm_names():
    from loongforge_b200.config import build as B
    import os
    out = []
    for name, rel in sorted(B._scan_model_yaml().items()):
        with open(os.path.join(B.CONFIG_DIR, rel)) as f:
            if "@model.image_encoder" in f.read():
                out.append(name)
    return out


@pytest.mark.parametrize("name", _vlm_names())
def test_every_vlm_yaml_builds_and_trains_at_reduced_size(name):
    """Every vision-language YAML under configs/models: composed, both towers shrunk to two layers of width 64 (all other
    architecture switches kept: norms, biases, position tables, MLA / MoE / hybrid layers of the language model), then one
    forward / backward through the composed model."""
    import dataclasses
    import os
    from loongforge_b200.config import build as B
    from loongforge_b200.config import yaml_compose
    from loongforge_b200.models.omni import OmniCombinationModel

    os.environ.setdefault("LOONGFORGE_PATH", B.REPO_ROOT)
    raw = yaml_compose.compose(os.path.join(B.CONFIG_DIR, B._scan_model_yaml()[name]))
    node = raw["model"]
    enc = node["image_encoder"]
    vit = B.transformer_config_from_yaml({k: v for k, v in enc.items() if not isinstance(v, dict) and k != "freeze"})
    vit = dataclasses.replace(vit, num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=4, kv_channels=16,
                              ffn_hidden_size=128)
    lm = B.transformer_config_from_yaml({k: v for k, v in node["foundation"].items() if not isinstance(v, dict)})
    small = dict(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, kv_channels=16, ffn_hidden_size=128,
                 vocab_size=300, make_vocab_size_divisible_by=1, mtp_num_layers=0)
    if lm.num_moe_experts:
        small.update(num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_layer_freq=[0, 1] if isinstance(lm.moe_layer_freq, list) else 1,
                     moe_router_num_groups=None, moe_router_group_topk=None)
        if lm.moe_shared_expert_intermediate_size:
            small["moe_shared_expert_intermediate_size"] = 32
    if lm.multi_latent_attention:
        small.update(q_lora_rank=24, kv_lora_rank=16, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16, kv_channels=None)
        if lm.use_dsa:
            small.update(dsa_indexer_n_heads=2, dsa_indexer_head_dim=16, dsa_indexer_topk=8, dsa_indexer_topk_freq=1,
                         dsa_indexer_skip_topk_offset=0)
    if lm.full_attention_interval:
        small.update(full_attention_interval=2, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                     linear_value_head_dim=16, kv_channels=16)
    if lm.position_embedding_type == "mrope":
        full = not lm.rotary_percent or lm.rotary_percent == 1.0
        small["mrope_section"] = [4, 2, 2] if full else [1, 1, 0]          # sums to (head channels x rotary share) / 2
        small["rotary_percent"] = 1.0 if full else 0.25
    lm = dataclasses.replace(lm, **small)
    family = str(enc.get("model_type", "qwen2_5_vit"))
    family = family if family in VZ.VISION_FAMILIES else "qwen2_vit"
    opts = dict(enc.get("vision_options") or {})
    if "pos_table_side" in opts:
        opts["pos_table_side"] = 8
    if "deepstack_indexes" in opts:
        opts["deepstack_indexes"] = (0, 1)
    torch.manual_seed(0)
    m = OmniCombinationModel(lm, vit, image_token_id=299, vision_family=family, vision_options=opts or None)
    merge = vit.spatial_merge_size
    n_img_tok = sum(int(t * (h // merge) * (w // merge)) for t, h, w in GRID.tolist())
    tokens = torch.cat([torch.randint(0, 298, (5,)), torch.full((n_img_tok,), 299), torch.randint(0, 298, (7,))])
    T = tokens.numel()
    pos = torch.arange(T) if lm.position_embedding_type != "mrope" else torch.arange(T)[None].expand(3, -1)
    loss = m(tokens, pos, pixels=_pixels(vit), grid_thw=GRID, labels=torch.roll(tokens, -1), loss_mask=torch.ones(T)).mean()
    loss.backward()
    assert torch.isfinite(loss), name
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in m.parameters())


def test_vlm_cli_with_lora_described_in_the_model_yaml(tmp_path):
    """`model.peft_config` of a composed VLM YAML (configs/models/lora/vlm_lora.yaml) gives the language model adapters
    and leaves the frozen encoder alone; the run trains through the CLI."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    y = tmp_path / "tiny_vl_lora.yaml"
    y.write_text(f"""
defaults:
  - {root}/configs/models/lora@model.peft_config: vlm_lora
  - _self_
model:
  model_type: qwen2_5_vl
  image_encoder:
    model_type: qwen2_5_vit
    freeze: true
    num_layers: 2
    hidden_size: 64
    kv_channels: 16
    ffn_hidden_size: 128
    num_attention_heads: 4
    num_query_groups: 4
    patch_size: 14
    temporal_patch_size: 2
    spatial_merge_size: 2
    normalization: RMSNorm
    add_qkv_bias: true
    causal: false
    vocab_size: 0
  foundation:
    model_type: llama
    num_layers: 2
    hidden_size: 64
    num_attention_heads: 4
    num_query_groups: 2
    ffn_hidden_size: 128
    vocab_size: 512
  peft_config:
    apply_to_foundation: true
    dim: 4
""")
    cmd = [sys.executable, "-m", "loongforge_b200.train", "--config-file", str(y), "--training-phase", "sft", "--mock-data",
           "--seq-length", "64", "--micro-batch-size", "1", "--global-batch-size", "2", "--train-iters", "2", "--lr", "1e-3",
           "--image-resolution", "56", "--log-interval", "1"]
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "iteration        2/" in p.stdout
    line = next(l for l in p.stdout.splitlines() if "LoRA adapters" in l)
    assert "foundation: 8 linears" in line and "image_encoder" not in line        # 2 layers x (qkv, proj, fc1, fc2)
    m = __import__("re").search(r"([\d,]+) trainable parameters of ([\d,]+)", line)
    trainable, total = (int(x.replace(",", "")) for x in m.groups())
    assert 0 < trainable < 0.6 * total            # adapters + the (unfrozen) projector; base language model and encoder are fixed


def test_vlm_cli_trains_on_shards_with_videos(tmp_path):
    """Shards that mix image samples and video samples (.mp4 members): the loader decodes --frame-num frames, the task
    encoder writes <video> placeholders, the trainer runs the vision tower over both kinds in one patch stream."""
    import json
    import os
    import subprocess
    import sys

    import cv2
    import numpy as np
    from tools.data_preprocess.vlm_to_webdataset import write_shards

    raw = tmp_path / "raw"
    raw.mkdir()
    rng = np.random.RandomState(0)
    recs = []
    for i in range(4):
        np.save(raw / f"{i}.npy", rng.randint(0, 255, size=(56, 56, 3), dtype=np.uint8))
        recs.append({"image": f"{i}.npy", "conversations": [{"from": "human", "value": "<image>what?"}, {"from": "gpt", "value": f"item {i}"}]})
        w = cv2.VideoWriter(str(raw / f"{i}.mp4"), cv2.VideoWriter_fourcc(*"mp4v"), 10, (56, 56))
        for t in range(8):
            w.write(rng.randint(0, 255, size=(56, 56, 3), dtype=np.uint8))
        w.release()
        recs.append({"video": f"{i}.mp4", "conversations": [{"from": "human", "value": "<video>what moves?"}, {"from": "gpt", "value": f"clip {i}"}]})
    write_shards(recs, str(tmp_path / "wds"), image_root=str(raw), samples_per_shard=4)
    y = tmp_path / "tiny_vl.yaml"
    y.write_text(json.dumps({"model": {
        "model_type": "qwen2_5_vl",
        "image_encoder": {"model_type": "qwen2_5_vit", "num_layers": 2, "hidden_size": 64, "kv_channels": 16, "ffn_hidden_size": 128,
                          "num_attention_heads": 4, "num_query_groups": 4, "patch_size": 14, "temporal_patch_size": 2,
                          "spatial_merge_size": 2, "causal": False, "vocab_size": 0, "fullatt_block_indexes": [1], "vision_window_size": 56},
        "foundation": {"model_type": "qwen2", "num_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_query_groups": 2,
                       "ffn_hidden_size": 128, "vocab_size": 512, "position_embedding_type": "mrope", "mrope_section": [2, 3, 3]}}}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "loongforge_b200.train", "--config-file", str(y), "--seq-length", "192", "--micro-batch-size", "1",
           "--global-batch-size", "2", "--train-iters", "3", "--lr", "1e-3", "--log-interval", "1", "--data-path", str(tmp_path / "wds"),
           "--training-phase", "sft", "--frame-num", "4"]
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "iteration        3/" in p.stdout and "lm loss" in p.stdout
