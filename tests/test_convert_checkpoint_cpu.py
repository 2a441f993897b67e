"""HF -> mcore (TP2 x PP2 / EP2) -> HF round trip is exact; the converted shards load into the model."""
import pytest
import json
import os

import torch


def _fake_hf(tmp, L=4, h=64, nh=4, ng=2, ffn=96, V=1000, experts=None, qk_norm=False, bias=False):
    from safetensors.torch import save_file

    torch.manual_seed(0)
    d = h // nh
    sd = {"model.embed_tokens.weight": torch.randn(V, h), "model.norm.weight": torch.randn(h),
          "lm_head.weight": torch.randn(V, h)}
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = torch.randn(h)
        sd[p + "post_attention_layernorm.weight"] = torch.randn(h)
        sd[p + "self_attn.q_proj.weight"] = torch.randn(nh * d, h)
        sd[p + "self_attn.k_proj.weight"] = torch.randn(ng * d, h)
        sd[p + "self_attn.v_proj.weight"] = torch.randn(ng * d, h)
        sd[p + "self_attn.o_proj.weight"] = torch.randn(h, nh * d)
        if bias:
            for n, r in (("q", nh), ("k", ng), ("v", ng)):
                sd[p + f"self_attn.{n}_proj.bias"] = torch.randn(r * d)
        if qk_norm:
            sd[p + "self_attn.q_norm.weight"] = torch.randn(d)
            sd[p + "self_attn.k_norm.weight"] = torch.randn(d)
        if experts:
            sd[p + "mlp.gate.weight"] = torch.randn(experts, h)
            for e in range(experts):
                q = p + f"mlp.experts.{e}."
                sd[q + "gate_proj.weight"], sd[q + "up_proj.weight"] = torch.randn(ffn, h), torch.randn(ffn, h)
                sd[q + "down_proj.weight"] = torch.randn(h, ffn)
        else:
            sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = torch.randn(ffn, h), torch.randn(ffn, h)
            sd[p + "mlp.down_proj.weight"] = torch.randn(h, ffn)
    os.makedirs(tmp, exist_ok=True)
    save_file(sd, os.path.join(tmp, "model.safetensors"))
    cfg = {"num_hidden_layers": L, "num_attention_heads": nh, "num_key_value_heads": ng, "vocab_size": V}
    if experts:
        cfg["num_experts"] = experts
    json.dump(cfg, open(os.path.join(tmp, "config.json"), "w"))
    return sd


def _roundtrip(tmp_path, family, extra, **hf_kw):
    from tools.convert_checkpoint import convert

    src = _fake_hf(str(tmp_path / "hf"), **hf_kw)
    convert.main(["--load_platform", "huggingface", "--save_platform", "mcore", "--model_type_custom", family,
                  "--load_ckpt_path", str(tmp_path / "hf"), "--save_ckpt_path", str(tmp_path / "mc"),
                  "--make_vocab_size_divisible_by", "64"] + extra)
    convert.main(["--load_platform", "mcore", "--save_platform", "huggingface", "--model_type_custom", family,
                  "--load_ckpt_path", str(tmp_path / "mc"), "--save_ckpt_path", str(tmp_path / "hf2"),
                  "--num_layers", str(hf_kw.get("L", 4)), "--num_attention_heads", "4", "--num_query_groups", "2",
                  "--vocab_size", "1000"] + (["--num_experts", str(hf_kw["experts"])] if hf_kw.get("experts") else []))
    from safetensors.torch import load_file

    back = load_file(str(tmp_path / "hf2" / "model.safetensors"))
    assert set(back) == set(src)
    for k in src:
        assert torch.equal(back[k], src[k]), k


def test_dense_tp2_pp2_roundtrip(tmp_path):
    _roundtrip(tmp_path, "qwen2", ["--tensor_model_parallel_size", "2", "--pipeline_model_parallel_size", "2"], bias=True)
    d = tmp_path / "mc" / "release"
    assert sorted(os.listdir(d)) == ["mp_rank_00_000", "mp_rank_00_001", "mp_rank_01_000", "mp_rank_01_001"]
    assert open(tmp_path / "mc" / "latest_checkpointed_iteration.txt").read() == "release"
    sd = torch.load(d / "mp_rank_01_001" / "model_optim_rng.pt", weights_only=False)["model"]
    assert "decoder.layers.0.self_attention.linear_qkv.weight" in sd and "embedding.word_embeddings.weight" not in sd
    assert sd["decoder.layers.1.mlp.linear_fc1.weight"].shape == (96, 64)  # [gate/2; up/2]
    assert sd["output_layer.weight"].shape == (1024 // 2, 64)  # vocab padded to 64*tp then sharded


def test_moe_ep2_roundtrip(tmp_path):
    _roundtrip(tmp_path, "qwen3_moe", ["--expert_parallel_size", "2"], experts=4, qk_norm=True)


def test_converted_checkpoint_loads_into_model(tmp_path):
    from tools.convert_checkpoint import convert
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.models.gpt import GPTModel

    src = _fake_hf(str(tmp_path / "hf"))
    convert.main(["--load_platform", "huggingface", "--save_platform", "mcore", "--model_type_custom", "llama3",
                  "--load_ckpt_path", str(tmp_path / "hf"), "--save_ckpt_path", str(tmp_path / "mc"),
                  "--make_vocab_size_divisible_by", "8"])
    sd = torch.load(tmp_path / "mc" / "release" / "mp_rank_00" / "model_optim_rng.pt", weights_only=False)["model"]
    cfg = TransformerConfig(num_layers=4, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                            ffn_hidden_size=96, vocab_size=1000, make_vocab_size_divisible_by=8)
    m = GPTModel(cfg)
    missing, unexpected = m.load_state_dict(sd, strict=True)
    assert not missing and not unexpected
    # logits equal those of a straight HF-style computation of the first layer's q projection path
    x = torch.randn(5, 64)
    q_hf = x @ src["model.layers.0.self_attn.q_proj.weight"].t()
    qkv = (x @ m.decoder.layers[0].self_attention.linear_qkv.weight.t()).view(5, 2, 4, 16)
    assert torch.allclose(qkv[:, :, :2].reshape(5, 64), q_hf, atol=1e-5)


def test_online_hf_bridge_roundtrip(tmp_path):
    from loongforge_b200.ckpt.hf_bridge import load_hf_checkpoint_online, save_hf_checkpoint
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer
    from safetensors.torch import load_file

    src = _fake_hf(str(tmp_path / "hf"))
    cfg = TransformerConfig(num_layers=4, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                            ffn_hidden_size=96, vocab_size=1000, make_vocab_size_divisible_by=8)
    tr = Trainer(cfg, TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=16, train_iters=1))
    assert load_hf_checkpoint_online(tr, str(tmp_path / "hf")) > 0
    save_hf_checkpoint(tr, str(tmp_path / "out"))
    back = load_file(str(tmp_path / "out" / "model.safetensors"))
    for k in src:
        assert torch.allclose(back[k], src[k], rtol=1e-4, atol=1e-6), k


def test_preprocess_and_log_parser(tmp_path):
    import json as js
    from tools.data_preprocess import preprocess_pretrain_data as pp
    from tools.log2json import parse
    from loongforge_b200.data.indexed_dataset import IndexedDataset

    p = tmp_path / "c.jsonl"
    p.write_text("\n".join(js.dumps({"text": "hello world %d" % i}) for i in range(5)))
    pp.main(["--input", str(p), "--output-prefix", str(tmp_path / "out" / "c"), "--append-eod"])
    ds = IndexedDataset(str(tmp_path / "out" / "c_text_document"))
    assert len(ds) == 5 and ds[0][-1] == 257
    line = (" [2026-01-01 00:00:00] iteration        3/      20 | consumed samples:           96 | elapsed time per "
            "iteration (ms): 4614.6 | throughput (token/sec/GPU): 3550.1 | learning rate: 1.0E-04 | global batch size:"
            "    32 | lm loss: 1.042075E+01 | loss scale: 1.0 | grad norm: 4.648900 |")
    rec = parse([line])[0]
    assert rec["iteration"] == 3 and rec["throughput"] == 3550.1 and abs(rec["lm_loss"] - 10.42075) < 1e-6


def test_deepseek_name_map_roundtrip_with_mtp_and_indexer():
    """MLA projections, lightning indexer, dense + MoE layers with shared expert and router bias, one MTP layer."""
    import torch

    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-deepseek", mtp_num_layers=1, moe_router_enable_expert_bias=True)
    mc = {k: v for k, v in build_model(cfg).state_dict().items() if "local_tokens_per_expert" not in k}
    kw = dict(num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads, num_groups=cfg.num_query_groups,
              num_experts=cfg.num_moe_experts)
    hf = nm.mcore_to_hf(mc, nm.FAMILIES["deepseek"], vocab_size=cfg.vocab_size, **kw)
    for name in ("model.layers.0.self_attn.q_a_proj.weight", "model.layers.0.self_attn.kv_a_proj_with_mqa.weight",
                 "model.layers.0.self_attn.kv_b_proj.weight", "model.layers.0.self_attn.indexer.wq_b.weight",
                 "model.layers.0.mlp.gate_proj.weight", "model.layers.1.mlp.gate.e_score_correction_bias",
                 "model.layers.1.mlp.experts.7.down_proj.weight", "model.layers.1.mlp.shared_experts.up_proj.weight",
                 "model.layers.2.eh_proj.weight", "model.layers.2.shared_head.norm.weight",
                 "model.layers.2.shared_head.head.weight", "model.layers.2.self_attn.q_b_proj.weight", "lm_head.weight"):
        assert name in hf, name
    back = nm.hf_to_mcore(hf, nm.FAMILIES["deepseek"], padded_vocab=cfg.padded_vocab_size, **kw)
    assert set(back) == set(mc)
    assert all(torch.equal(back[k], mc[k]) for k in mc)
    # tensor-parallel sharding rules of the MLA projections survive a split / merge
    for key in ("decoder.layers.0.self_attention.linear_q_up_proj.weight",
                "decoder.layers.0.self_attention.linear_kv_up_proj.weight", "mtp.layers.0.eh_proj.weight",
                "decoder.layers.1.mlp.shared_experts.linear_fc1.weight"):
        parts = [nm.shard_tp(key, mc[key], r, 2) for r in range(2)]
        assert parts[0].shape[0] * 2 == mc[key].shape[0] and torch.equal(nm.merge_tp(key, parts), mc[key])


def _ds_bridge(rank, world, tmp, dims_kw, mode):
    import os

    from loongforge_b200.ckpt.hf_bridge import load_hf_checkpoint_online, save_hf_checkpoint
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-deepseek", mtp_num_layers=1, moe_aux_loss_coeff=0.0)
    cfg.sequence_parallel = dims_kw.get("tp", 1) > 1
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=4, lr=1e-3, clip_grad=1.0,
                     log_interval=1000)
    tr = Trainer(cfg, tc, ParallelDims(**dims_kw))
    st = tr.st
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=3, pin_memory=False)
    if mode == "save":
        for _ in range(2):
            tr.train_step(it)
        save_hf_checkpoint(tr, os.path.join(tmp, "hf"), family="deepseek")
    else:
        load_hf_checkpoint_online(tr, os.path.join(tmp, "hf"), family="deepseek")
        for _ in range(2 * 4 // st.dp_size):
            next(it)
    m = tr.train_step(it)
    return m.get("lm loss"), m["grad_norm"]


def test_deepseek_online_bridge_across_layouts(tmp_path):
    from dist_utils import run_distributed

    a = run_distributed(_ds_bridge, 2, str(tmp_path), {"tp": 2}, "save")
    b = run_distributed(_ds_bridge, 2, str(tmp_path), {"ep": 2}, "load")
    assert abs(a[0][0] - b[0][0]) < 1e-4 * a[0][0] and abs(a[0][1] - b[0][1]) < 1e-3 * max(1, a[0][1]), (a, b)


def test_qwen_vl_name_map_roundtrip_and_numerics():
    """Vision tower + merger + language model of the Qwen2.5-VL layout: names round-trip, and the per-head QKV
    packing reproduces the fused [q; k; v] projection."""
    import torch

    from loongforge_b200.models.omni import OmniCombinationModel
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    lm = get_model_config("tiny-llama", add_qkv_bias=True, position_embedding_type="mrope", mrope_section=[8, 12, 12])
    vit = get_model_config("tiny-vit")
    model = OmniCombinationModel(lm, vit, image_token_id=lm.vocab_size - 1)
    mc = dict(model.state_dict())
    kw = dict(vit_layers=vit.num_layers, vit_heads=vit.num_attention_heads, num_layers=lm.num_layers,
              num_heads=lm.num_attention_heads, num_groups=lm.num_query_groups)
    for nested in (False, True):
        hf = nm.vlm_mcore_to_hf(mc, nm.FAMILIES["qwen2.5"], nested=nested, vocab_size=lm.vocab_size, **kw)
        vp = "model.visual." if nested else "visual."
        assert vp + "blocks.1.attn.qkv.bias" in hf and vp + "merger.mlp.2.weight" in hf
        assert ("model.language_model.layers.0.self_attn.q_proj.bias" if nested else "model.layers.0.self_attn.q_proj.bias") in hf
        back = nm.vlm_hf_to_mcore(hf, nm.FAMILIES["qwen2.5"], padded_vocab=lm.padded_vocab_size, **kw)
        assert set(back) == set(mc) and all(torch.equal(back[k], mc[k]) for k in mc)
    # fused HF projection == per-head packed Megatron projection, head by head
    H, d = vit.num_attention_heads, vit.kv_channels
    w = hf[vp + "blocks.0.attn.qkv.weight"]
    x = torch.randn(5, w.shape[1])
    q, k, v = (x @ w.t()).view(5, 3, H, d).unbind(1)
    packed = (x @ mc["encoder_model.image_encoder.decoder.layers.0.self_attention.linear_qkv.weight"].t()).view(5, H, 3, d)
    assert torch.allclose(packed[:, :, 0], q, atol=1e-6) and torch.allclose(packed[:, :, 2], v, atol=1e-6)


def test_converter_cli_vlm_roundtrip_with_tp_pp(tmp_path):
    """HF Qwen2.5-VL layout -> Megatron (TP 2, PP 2; encoder on the first stage) -> HF: bit-identical."""
    import json

    import torch

    from loongforge_b200.models.omni import OmniCombinationModel
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import convert as C
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    lm = get_model_config("tiny-llama", add_qkv_bias=True, position_embedding_type="mrope", mrope_section=[8, 12, 12])
    vit = get_model_config("tiny-vit")
    mc = dict(OmniCombinationModel(lm, vit, image_token_id=lm.vocab_size - 1).state_dict())
    kw = dict(vit_layers=vit.num_layers, vit_heads=vit.num_attention_heads, num_layers=lm.num_layers,
              num_heads=lm.num_attention_heads, num_groups=lm.num_query_groups)
    hf = nm.vlm_mcore_to_hf(mc, nm.FAMILIES["qwen2.5"], vocab_size=lm.vocab_size, **kw)
    cfg = {"model_type": "qwen2_5_vl", "text_config": {"num_hidden_layers": lm.num_layers, "vocab_size": lm.vocab_size,
                                                        "num_attention_heads": lm.num_attention_heads,
                                                        "num_key_value_heads": lm.num_query_groups},
           "vision_config": {"depth": vit.num_layers, "num_heads": vit.num_attention_heads}}
    C.save_hf(hf, str(tmp_path / "hf"), cfg)
    common = ["--model_type_custom", "qwen2_5_vl", "--vit_num_heads", str(vit.num_attention_heads)]
    C.main(["--load_platform", "huggingface", "--save_platform", "mcore", "--load_ckpt_path", str(tmp_path / "hf"),
            "--save_ckpt_path", str(tmp_path / "mc"), "--tensor_model_parallel_size", "2",
            "--pipeline_model_parallel_size", "2"] + common)
    first = torch.load(tmp_path / "mc" / "release" / "mp_rank_00_000" / "model_optim_rng.pt", weights_only=False)["model"]
    last = torch.load(tmp_path / "mc" / "release" / "mp_rank_01_001" / "model_optim_rng.pt", weights_only=False)["model"]
    assert any(k.startswith("encoder_model.image_encoder") for k in first) and not any(k.startswith("encoder_model") for k in last)
    assert "foundation_model.decoder.layers.0.mlp.linear_fc2.weight" in last and "foundation_model.output_layer.weight" in last
    C.main(["--load_platform", "mcore", "--save_platform", "huggingface", "--load_ckpt_path", str(tmp_path / "mc"),
            "--save_ckpt_path", str(tmp_path / "back"), "--num_layers", str(lm.num_layers), "--num_attention_heads",
            str(lm.num_attention_heads), "--num_query_groups", str(lm.num_query_groups), "--vocab_size",
            str(lm.vocab_size)] + common)
    back = C.load_hf(str(tmp_path / "back"))
    assert set(back) == set(hf) and all(torch.equal(back[k], hf[k]) for k in hf)


def _dist_ckpt_worker(rank, world, tmp, dims_kw, mode):
    import os

    from loongforge_b200.ckpt.hf_bridge import save_hf_checkpoint
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-llama")
    cfg.sequence_parallel = dims_kw.get("tp", 1) > 1
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=4, lr=1e-3, log_interval=1000)
    tr = Trainer(cfg, tc, ParallelDims(**dims_kw))
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, seed=3, pin_memory=False)
    if mode == "save":
        for _ in range(2):
            tr.train_step(it)
        tr.save_checkpoint(os.path.join(tmp, "ck"))
        save_hf_checkpoint(tr, os.path.join(tmp, "hf_online"), family="llama3")
    else:
        tr.load_checkpoint(os.path.join(tmp, "ck2"), load_optim=False, load_rng=False)
        for _ in range(8):
            next(it)
    return tr.train_step(it).get("lm loss")


def test_offline_dist_checkpoint_to_hf_and_back(tmp_path):
    """torch_dist checkpoint written under TP 2 -> HF files offline (equal to the online export) -> weights-only
    torch_dist checkpoint offline -> loaded under PP 2: the next loss is the one of the run that saved."""
    import torch

    from dist_utils import run_distributed
    from tools.convert_checkpoint.convert import load_hf
    from tools.dist_checkpoint import convert_dist_checkpoint as T

    a = run_distributed(_dist_ckpt_worker, 2, str(tmp_path), {"tp": 2}, "save")
    assert T.main(["--to", "hf", "--load", str(tmp_path / "ck"), "--save", str(tmp_path / "hf"), "--family", "llama3"]) == 0
    off, on = load_hf(str(tmp_path / "hf")), load_hf(str(tmp_path / "hf_online"))
    assert set(off) == set(on) and all(torch.equal(off[k], on[k]) for k in on)
    assert (tmp_path / "hf" / "config.json").is_file()
    assert T.main(["--to", "dist", "--load", str(tmp_path / "hf"), "--save", str(tmp_path / "ck2"), "--family", "llama3",
                   "--model-name", "tiny-llama"]) == 0
    b = run_distributed(_dist_ckpt_worker, 2, str(tmp_path), {"pp": 2}, "load")
    assert abs(a[0] - b[1]) < 1e-5 * a[0], (a, b)


def test_family_spellings_internlm2_minimax_mimo_roundtrip():
    """Families whose Hugging Face files name the same tensors differently: packed wqkv + w1/w3/w2 (InternLM2),
    block_sparse_moe with a router bias (MiniMax), MTP layers under model.mtp_layers (MiMo)."""
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cases = {
        "internlm2": (get_model_config("tiny-llama"),
                      ["model.tok_embeddings.weight", "output.weight", "model.layers.0.attention.wqkv.weight",
                       "model.layers.0.attention.wo.weight", "model.layers.1.feed_forward.w3.weight",
                       "model.layers.1.attention_norm.weight", "model.layers.1.ffn_norm.weight"]),
        "minimax": (get_model_config("tiny-qwen3-moe", moe_router_enable_expert_bias=True),
                    ["model.layers.0.block_sparse_moe.gate.weight", "model.layers.0.block_sparse_moe.experts.3.w1.weight",
                     "model.layers.0.block_sparse_moe.experts.3.w2.weight",
                     "model.layers.0.block_sparse_moe.e_score_correction_bias", "model.layers.0.self_attn.q_norm.weight"]),
        "mimo": (get_model_config("tiny-llama", add_qkv_bias=True, mtp_num_layers=1),
                 ["model.mtp_layers.0.token_layernorm.weight", "model.mtp_layers.0.hidden_layernorm.weight",
                  "model.mtp_layers.0.input_proj.weight", "model.mtp_layers.0.final_layernorm.weight",
                  "model.mtp_layers.0.self_attn.q_proj.bias", "model.mtp_layers.0.mlp.down_proj.weight"]),
    }
    for family, (cfg, expect) in cases.items():
        fam = nm.FAMILIES[family]
        mc = {k: v for k, v in build_model(cfg).state_dict().items()
              if "local_tokens_per_expert" not in k and "_extra_state" not in k}
        kw = dict(num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads, num_groups=cfg.num_query_groups,
                  num_experts=cfg.num_moe_experts)
        hf = nm.mcore_to_hf(mc, fam, vocab_size=cfg.vocab_size, **kw)
        for name in expect:
            assert name in hf, (family, name, sorted(hf)[:12])
        assert not any("self_attn.wqkv" in k or ".gate_proj." in k and family == "minimax" for k in hf), family
        back = nm.hf_to_mcore(hf, fam, padded_vocab=cfg.padded_vocab_size, **kw)
        assert set(back) == set(mc), (family, set(back) ^ set(mc))
        assert all(torch.equal(back[k], mc[k]) for k in mc), family
    ps.destroy_model_parallel()


def _hybrid_shard_worker(rank, world, tmp):
    """The TP shard that the converter cuts equals what a TP rank of the model itself holds."""
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    cfg = get_model_config("tiny-qwen3-next")
    nm.set_linear_attention_geometry(cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_num_value_heads,
                                     cfg.linear_value_head_dim)
    full = torch.load(os.path.join(tmp, "full.pt"))
    ps.initialize_model_parallel(ps.ParallelDims(tp=2))
    local = build_model(cfg).state_dict()
    bad = [k for k, w in full.items() if k in local and not torch.equal(nm.shard_tp(k, w, rank, 2), local[k])]
    return bad


def test_qwen3_next_name_map_roundtrip_and_tp_shards(tmp_path):
    """GatedDeltaNet + gated attention + gated shared expert: names, the per-head [q; gate] packing, TP rules."""
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from tests.dist_utils import run_distributed
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-qwen3-next", mtp_num_layers=1)
    fam = nm.FAMILIES["qwen3_next"]
    mc = {k: v for k, v in build_model(cfg).state_dict().items()
          if "local_tokens_per_expert" not in k and "_extra_state" not in k and "expert_bias" not in k}
    kw = dict(num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads, num_groups=cfg.num_query_groups,
              num_experts=cfg.num_moe_experts)
    hf = nm.mcore_to_hf(mc, fam, vocab_size=cfg.vocab_size, **kw)
    d, nh = cfg.kv_channels, cfg.num_attention_heads
    assert hf["model.layers.3.self_attn.q_proj.weight"].shape == (2 * nh * d, cfg.hidden_size)
    assert hf["model.layers.0.linear_attn.conv1d.weight"].dim() == 3
    for name in ("model.layers.0.linear_attn.in_proj_qkvz.weight", "model.layers.0.linear_attn.A_log",
                 "model.layers.0.linear_attn.norm.weight", "model.layers.0.mlp.shared_expert_gate.weight",
                 "model.layers.0.mlp.shared_expert.down_proj.weight", "model.layers.3.self_attn.k_norm.weight",
                 "mtp.fc.weight", "mtp.pre_fc_norm_hidden.weight", "mtp.norm.weight",
                 "mtp.layers.0.self_attn.q_proj.weight", "mtp.layers.0.mlp.shared_expert_gate.weight"):
        assert name in hf, name
    # head 1's query rows sit at [2 d, 3 d) of the HF projection and in group 0's q block of the packed one
    packed = mc["decoder.layers.3.self_attention.linear_qgkv.weight"]
    assert torch.equal(hf["model.layers.3.self_attn.q_proj.weight"][2 * d:3 * d], packed[d:2 * d])
    back = nm.hf_to_mcore(hf, fam, padded_vocab=cfg.padded_vocab_size, **kw)
    assert set(back) == set(mc), set(back) ^ set(mc)
    assert all(torch.equal(back[k], mc[k]) for k in mc)
    nm.set_linear_attention_geometry(cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_num_value_heads,
                                     cfg.linear_value_head_dim)
    for k, w in mc.items():
        assert torch.equal(nm.merge_tp(k, [nm.shard_tp(k, w, r, 2) for r in range(2)]), w), k
    torch.save(mc, tmp_path / "full.pt")
    ps.destroy_model_parallel()
    for bad in run_distributed(_hybrid_shard_worker, 2, str(tmp_path)):
        assert not bad, bad


def _minimax_shard_worker(rank, world, tmp):
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    cfg = get_model_config("tiny-minimax")
    nm.set_qk_norm_over_all_heads(cfg.qk_layernorm_full)
    full = torch.load(os.path.join(tmp, "full.pt"))
    ps.initialize_model_parallel(ps.ParallelDims(tp=2))
    local = build_model(cfg).state_dict()
    return [k for k, w in full.items() if k in local and ".experts." not in k
            and nm.shard_tp(k, w, rank, 2).shape != local[k].shape]


def test_minimax_full_head_qk_norm_is_split_with_the_heads(tmp_path):
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    from tests.dist_utils import run_distributed

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    mc = {k: v for k, v in build_model(get_model_config("tiny-minimax")).state_dict().items() if "_extra_state" not in k}
    torch.save(mc, tmp_path / "full.pt")
    ps.destroy_model_parallel()
    for bad in run_distributed(_minimax_shard_worker, 2, str(tmp_path)):
        assert not bad, bad


def test_qwen3_vl_vision_tower_and_deepstack_name_map_roundtrip():
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.models.vision_zoo import DeepStackMergers, build_vision_encoder
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = get_model_config("tiny-vit")
    vit = {k: v for k, v in build_vision_encoder("qwen3_vl_vit", cfg, deepstack_indexes=(0, 1)).state_dict().items()
           if "_extra_state" not in k}
    taps = dict(DeepStackMergers(cfg, 96, 2).state_dict())
    hf = nm.qwen3_vision_to_hf(vit, taps, num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads)
    for name in ("model.visual.pos_embed.weight", "model.visual.blocks.0.attn.qkv.weight", "model.visual.blocks.1.norm2.weight",
                 "model.visual.blocks.0.mlp.linear_fc1.bias", "model.visual.deepstack_merger_list.1.norm.bias",
                 "model.visual.deepstack_merger_list.0.linear_fc2.weight"):
        assert name in hf, name
    d = cfg.hidden_size // cfg.num_attention_heads
    # HF rows are [q of all heads; k of all heads; v of all heads]; ours are per head [q_h, k_h, v_h]
    assert torch.equal(hf["model.visual.blocks.0.attn.qkv.weight"][d:2 * d],
                       vit["decoder.layers.0.self_attention.linear_qkv.weight"][3 * d:4 * d])
    vit2, taps2 = nm.qwen3_vision_to_mcore(hf, num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads)
    assert set(vit2) == set(vit) and all(torch.equal(vit2[k], vit[k]) for k in vit)
    assert set(taps2) == set(taps) and all(torch.equal(taps2[k], taps[k]) for k in taps)
    ps.destroy_model_parallel()


def test_online_upcycling_from_a_dense_hf_checkpoint(tmp_path):
    """--moe-use-upcycling: a dense HF checkpoint initialises an MoE model whose output equals the dense model's
    (4 experts of half the dense width, top-2 over distinct slices is not guaranteed by a random router, so the
    check is on the weights: every expert is a slice of the dense FFN, FC2 scaled by the granularity)."""
    from loongforge_b200.ckpt.hf_bridge import load_hf_checkpoint_online
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    ps.destroy_model_parallel()
    src = _fake_hf(str(tmp_path / "hf"), L=2, ffn=128)
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=128,
                            vocab_size=1000, make_vocab_size_divisible_by=8, num_moe_experts=4, moe_router_topk=2,
                            moe_ffn_hidden_size=64)
    tr = Trainer(cfg, TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=16, train_iters=1))
    assert load_hf_checkpoint_online(tr, str(tmp_path / "hf"), upcycle=True) > 0
    sd = tr.models[0].module.state_dict()
    gate, up = src["model.layers.1.mlp.gate_proj.weight"], src["model.layers.1.mlp.up_proj.weight"]
    down = src["model.layers.1.mlp.down_proj.weight"]
    for e in range(4):
        s = e % 2
        fc1 = sd[f"decoder.layers.1.mlp.experts.linear_fc1.weight{e}"].float()
        fc2 = sd[f"decoder.layers.1.mlp.experts.linear_fc2.weight{e}"].float()
        assert torch.allclose(fc1, torch.cat([gate[s * 64:(s + 1) * 64], up[s * 64:(s + 1) * 64]]), atol=1e-6)
        assert torch.allclose(fc2, down[:, s * 64:(s + 1) * 64] * 2, atol=1e-6)
    assert torch.allclose(sd["decoder.layers.1.pre_mlp_layernorm.weight"].float(),
                          src["model.layers.1.post_attention_layernorm.weight"])
    assert sd["decoder.layers.0.mlp.router.weight"].shape == (4, 64)
    ps.destroy_model_parallel()


@pytest.mark.parametrize("family", ["intern_vit", "moon_vit"])
def test_generic_vision_tower_name_maps_round_trip(family):
    """InternViT / MoonViT towers with their projectors: every tensor of the built modules has a public name, the shapes on
    the public side are the published ones (Conv2d patch weight, [1, 1 + N, C] or [H, W, C] position table), and loading
    the converted tensors back reproduces the module's output."""
    import torch
    from loongforge_b200.models import vision_zoo as VZ
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, kv_channels=16, ffn_hidden_size=128, vocab_size=0,
                            normalization="LayerNorm", activation="gelu", gated_linear_unit=False, add_bias_linear=True, add_qkv_bias=True,
                            causal=False, patch_size=14, temporal_patch_size=1, spatial_merge_size=2, position_embedding_type="none",
                            qk_layernorm_full=(family == "intern_vit"))
    torch.manual_seed(0)
    vit = VZ.build_vision_encoder(family, cfg, pos_table_side=4)
    adapter = VZ.VISION_FAMILIES[family][1](cfg, 96)
    for p in list(vit.parameters()) + list(adapter.parameters()):
        torch.nn.init.normal_(p, std=0.05)
    mc = {"image_encoder." + k: v.detach().clone() for k, v in vit.state_dict().items()}
    mc.update({"image_projector." + k: v.detach().clone() for k, v in adapter.state_dict().items()})
    hf = nm.generic_vision_to_hf(mc, family, 2, 4)
    assert len(hf) == len(mc), sorted(set(mc) - {("image_encoder." + a) for a, _ in nm._GENERIC_VIT[family]["top"]})[:3]
    if family == "intern_vit":
        assert hf["vision_model.embeddings.patch_embedding.weight"].shape == (64, 3, 14, 14)
        assert hf["vision_model.embeddings.position_embedding"].shape == (1, 17, 64)
        assert hf["vision_model.embeddings.class_embedding"].shape == (1, 1, 64) and "mlp1.3.weight" in hf
        assert "vision_model.encoder.layers.1.attn.q_norm.weight" in hf and "vision_model.encoder.layers.0.ls2" in hf
    else:
        assert hf["vision_tower.patch_embed.pos_emb.weight"].shape == (4, 4, 64)
        assert "vision_tower.encoder.blocks.1.wqkv.bias" in hf and "multi_modal_projector.linear_2.weight" in hf
    # q rows of head 0 come first on the public side, per-head interleaved on ours
    w_pub = hf[("vision_model.encoder.layers.0.attn.qkv.weight" if family == "intern_vit" else "vision_tower.encoder.blocks.0.wqkv.weight")]
    w_own = mc["image_encoder.decoder.layers.0.self_attention.linear_qkv.weight"]
    assert torch.equal(w_pub[:16], w_own[:16]) and torch.equal(w_pub[64:80], w_own[16:32])
    back = nm.generic_vision_to_mcore(hf, family, 2, 4)
    assert set(back) == set(mc) and all(torch.equal(back[k], mc[k]) for k in mc)
    vit2 = VZ.build_vision_encoder(family, cfg, pos_table_side=4)
    vit2.load_state_dict({k[len("image_encoder."):]: v for k, v in back.items() if k.startswith("image_encoder.")})
    grid = torch.tensor([[1, 4, 4]])
    px = torch.randn(16, 3 * 14 * 14)
    assert torch.allclose(vit(px, grid)[0], vit2(px, grid)[0])


def test_internvl_style_checkpoint_converts_both_ways(tmp_path):
    """``language_model.*`` + ``vision_model.*`` + ``mlp1.*`` (InternVL layout, Qwen3 language model) -> TP2 training shards
    -> back: every tensor returns bit-exact."""
    from safetensors.torch import load_file, save_file
    from tools.convert_checkpoint import convert as C

    src = tmp_path / "lm"
    _fake_hf(str(src), L=2, V=512, qk_norm=True)
    lm = load_file(str(src / "model.safetensors"))
    torch.manual_seed(1)
    sd = {"language_model." + k: v for k, v in lm.items()}
    C_, nh = 64, 4
    sd.update({"vision_model.embeddings.class_embedding": torch.randn(1, 1, C_), "vision_model.embeddings.position_embedding": torch.randn(1, 17, C_),
               "vision_model.embeddings.patch_embedding.weight": torch.randn(C_, 3, 14, 14), "vision_model.embeddings.patch_embedding.bias": torch.randn(C_),
               "mlp1.0.weight": torch.randn(4 * C_), "mlp1.0.bias": torch.randn(4 * C_), "mlp1.1.weight": torch.randn(64, 4 * C_),
               "mlp1.1.bias": torch.randn(64), "mlp1.3.weight": torch.randn(64, 64), "mlp1.3.bias": torch.randn(64)})
    for i in range(2):
        p = f"vision_model.encoder.layers.{i}."
        sd.update({p + "norm1.weight": torch.randn(C_), p + "norm1.bias": torch.randn(C_), p + "norm2.weight": torch.randn(C_), p + "norm2.bias": torch.randn(C_),
                   p + "attn.qkv.weight": torch.randn(3 * C_, C_), p + "attn.qkv.bias": torch.randn(3 * C_), p + "attn.proj.weight": torch.randn(C_, C_),
                   p + "attn.proj.bias": torch.randn(C_), p + "ls1": torch.randn(C_), p + "ls2": torch.randn(C_), p + "mlp.fc1.weight": torch.randn(128, C_),
                   p + "mlp.fc1.bias": torch.randn(128), p + "mlp.fc2.weight": torch.randn(C_, 128), p + "mlp.fc2.bias": torch.randn(C_)})
    hf_dir = tmp_path / "internvl"
    os.makedirs(hf_dir)
    save_file(sd, str(hf_dir / "model.safetensors"))
    (hf_dir / "config.json").write_text(json.dumps({"llm_config": {"num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 512},
                                                    "vision_config": {"num_hidden_layers": 2, "num_attention_heads": nh}}))
    mc_dir, back_dir = tmp_path / "mc", tmp_path / "back"
    common = ["--model_type_custom", "internvl3.5", "--language_family", "qwen3", "--vit_num_heads", "4", "--num_layers", "2",
              "--num_attention_heads", "4", "--num_query_groups", "2", "--vocab_size", "512"]
    C.main(["--load_platform", "huggingface", "--save_platform", "mcore", "--load_ckpt_path", str(hf_dir), "--save_ckpt_path", str(mc_dir),
            "--tensor_model_parallel_size", "2", "--safetensors"] + common)
    C.main(["--load_platform", "mcore", "--save_platform", "huggingface", "--load_ckpt_path", str(mc_dir), "--save_ckpt_path", str(back_dir),
            "--safetensors"] + common)
    out = load_file(str(back_dir / "model.safetensors"))
    assert set(out) == set(sd), (sorted(set(sd) - set(out))[:4], sorted(set(out) - set(sd))[:4])
    assert all(torch.equal(out[k], sd[k]) for k in sd)
    with pytest.raises(SystemExit):
        C.main(["--load_platform", "huggingface", "--save_platform", "mcore", "--load_ckpt_path", str(hf_dir), "--save_ckpt_path", str(mc_dir),
                "--model_type_custom", "internvl"])
