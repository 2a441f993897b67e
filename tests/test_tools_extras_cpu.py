"""Converter formats (FP8 block, INT4 compressed-tensors, MXFP4), merge tools, SFT pre-tokenisation, offline packing,
WebDataset shards."""
import json
import os

import pytest
import torch


def test_fp8_block_format_roundtrip_with_ragged_edges():
    from tools.convert_checkpoint import quant_formats as Q

    torch.manual_seed(0)
    w = torch.randn(200, 300) * 3
    q, s = Q.fp8_block_quantize(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    back = Q.fp8_block_dequantize(q, s, dtype=torch.float32)
    assert ((back - w).abs() / w.abs().max()).max() < 0.04
    sd = {"a.weight": w, "model.norm.weight": torch.ones(300), "embed.weight": torch.randn(10, 4)}
    qsd = Q.quantize_fp8_state_dict(sd)
    assert "a.weight_scale_inv" in qsd and qsd["embed.weight"].dtype == torch.float32
    dsd = Q.dequantize_fp8_state_dict(qsd, dtype=torch.float32)
    assert set(dsd) == set(sd) and torch.allclose(dsd["a.weight"], back)


def test_int4_and_mxfp4():
    from tools.convert_checkpoint import quant_formats as Q

    torch.manual_seed(1)
    w = torch.randn(16, 256)
    for sym in (True, False):
        p, s, z = Q.int4_pack(w, 128, symmetric=sym)
        assert p.dtype == torch.int32 and p.shape == (16, 32) and s.shape == (16, 2) and (z is None) == sym
        back = Q.int4_unpack(p, s, z, 128, dtype=torch.float32)
        assert (back - w).abs().max() <= s.max() * 0.51 + 1e-6
    exact = torch.tensor([[0.5, -6.0, 3.0, 1.5] * 8]) * 4.0  # representable values with a shared exponent
    b, e = Q.mxfp4_quantize(exact)
    assert b.shape == (1, 1, 16) and e.shape == (1, 1)
    assert torch.equal(Q.mxfp4_dequantize(b, e, torch.float32), exact)
    r = torch.randn(4, 64)
    rb = Q.mxfp4_dequantize(*Q.mxfp4_quantize(r), torch.float32)
    assert ((rb - r).abs() / r.abs().amax(-1, keepdim=True)).max() < 0.26


def test_merge_tools():
    from tools.convert_checkpoint import merge_tools as M

    base = {"l.q_proj.weight": torch.zeros(4, 6), "other": torch.ones(1)}
    A, B = torch.randn(2, 6), torch.randn(4, 2)
    lora = {"base_model.model.l.q_proj.lora_A.default.weight": A, "base_model.model.l.q_proj.lora_B.default.weight": B}
    out = M.merge_lora_state_dict(base, lora, alpha=4, rank=2)
    assert torch.allclose(out["l.q_proj.weight"], 2.0 * B @ A) and torch.equal(out["other"], base["other"])
    vlm = M.merge_vlm_state_dicts({"a": torch.ones(1)}, {"b": torch.ones(1)}, {"c": torch.ones(1)})
    assert set(vlm) == {"foundation_model.a", "encoder_model.image_encoder.b", "encoder_model.image_projector.c"}
    s0 = {"x.experts.linear_fc1.weight0": torch.zeros(1), "x.experts.linear_fc1.weight1": torch.ones(1), "r": torch.ones(2)}
    s1 = {"x.experts.linear_fc1.weight0": torch.full((1,), 2.0), "x.experts.linear_fc1.weight1": torch.full((1,), 3.0),
          "r": torch.ones(2)}
    m = M.merge_expert_shards([s0, s1])
    assert [float(m[f"x.experts.linear_fc1.weight{i}"]) for i in range(4)] == [0, 1, 2, 3]


def test_sft_pretokenise_then_offline_packing(tmp_path):
    from tools.data_preprocess import offline_packing, preprocess_sft_data

    recs = [{"instruction": "say " + "x" * n, "output": "ok"} for n in (5, 50, 500, 20, 200, 3000)]
    src = tmp_path / "sft.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in recs))
    kept, dropped = preprocess_sft_data.main(["--input", str(src), "--output-path", str(tmp_path / "tok"),
                                              "--seq-length", "1000", "--shard-size", "3", "--enable-discard-sample"])
    assert (kept, dropped) == (5, 1)
    idx = json.load(open(tmp_path / "tok" / "index.json"))["splits"]["train"]
    assert len(idx["shards"]) == 2 and len(idx["lengths"]) == 5
    first = json.loads(open(tmp_path / "tok" / "train_00000.jsonl").readline())
    assert len(first["input_ids"]) == len(first["labels"]) and -100 in first["labels"]
    packs = offline_packing.main(["--index", str(tmp_path / "tok" / "index.json"), "--seq-length", "1000", "--output",
                                  str(tmp_path / "packs.json")])
    flat = sorted(i for p in packs for i in p)
    assert flat == [0, 1, 2, 3, 4]
    assert all(sum(idx["lengths"][i] for i in p) <= 1000 for p in packs) and len(packs) <= 3
    big = offline_packing.pack_with_buckets([700, 600, 300, 400, 100, 900, 50, 50], 1000, 64)
    assert sorted(i for p in big for i in p) == list(range(8)) and len(big) <= 4


def test_webdataset_shards(tmp_path):
    from tools.data_preprocess import vlm_to_webdataset as W

    (tmp_path / "img").mkdir()
    for i in range(3):
        (tmp_path / "img" / f"{i}.jpg").write_bytes(bytes([i]) * 10)
    recs = [{"image": f"{i}.jpg", "conversations": [{"from": "human", "value": "<image> hi"}]} for i in range(3)]
    recs.append({"image": ["0.jpg", "1.jpg"], "conversations": []})
    index = W.write_shards(recs, str(tmp_path / "wds"), str(tmp_path / "img"), samples_per_shard=3)
    assert index["total"] == 4 and [s["count"] for s in index["shards"]] == [3, 1]
    groups = list(W.read_shard(str(tmp_path / "wds" / "shard-000000.tar")))
    assert len(groups) == 3 and groups[1][1]["jpg"] == bytes([1]) * 10
    assert json.loads(groups[0][1]["json"])["num_images"] == 1
    multi = list(W.read_shard(str(tmp_path / "wds" / "shard-000001.tar")))[0][1]
    assert set(multi) == {"0.jpg", "1.jpg", "json"}


def test_layer_benchmark_exports_policy(tmp_path):
    from loongforge_b200.runtime.fp8_policy import FP8Policy
    from tools import benchmark_parallel_layers as B

    shapes = B.layer_shapes(__import__("loongforge_b200.models.registry", fromlist=["x"]).get_model_config("llama3-8b"), 2)
    assert shapes["linear_qkv"] == (4096, 3072) and shapes["linear_fc1"] == (4096, 14336) and shapes["linear_fc2"] == (7168, 4096)
    rows = B.run("tiny-llama", 1, [16, 32], warmup=1, iters=1)
    assert {r["kind"] for r in rows} == {"linear_qkv", "linear_proj", "linear_fc1", "linear_fc2", "output_layer"}
    assert len(rows) == 10 and all(r["bf16_ms"] > 0 and r["bf16_fwd_ms"] > 0 for r in rows)  # no ordering: the timings are noisy on a loaded host
    # multi-latent attention, routed (grouped) and shared experts, several tensor-parallel sizes in one sweep
    ds = B.layer_shapes(__import__("loongforge_b200.models.registry", fromlist=["x"]).get_model_config("deepseek-v3"), 2, ep=8)
    assert ds["linear_q_up_proj"] == (1536, 128 * 192 // 2) and ds["linear_kv_down_proj"] == (7168, 576)
    assert ds["experts.linear_fc1"] == (7168, 4096, 32) and ds["shared_experts.linear_fc2"] == (1024, 7168)
    rows = B.run("tiny-deepseek", [1, 2], [32], warmup=1, iters=1, kinds=["experts.linear_fc1", "linear_kv_up_proj"])
    assert {(r["kind"], r["tp"]) for r in rows} == {("experts.linear_fc1", 1), ("experts.linear_fc1", 2),
                                                    ("linear_kv_up_proj", 1), ("linear_kv_up_proj", 2)}
    assert all(r["experts"] == 8 for r in rows if r["kind"].startswith("experts"))
    out = tmp_path / "policy.json"
    B.main(["--model-name", "tiny-llama", "--tokens", "16", "--out", str(out), "--csv", str(tmp_path / "r.csv"),
            "--markdown", str(tmp_path / "r.md"), "--iters", "1", "--warmup", "1"])
    FP8Policy.from_json(str(out))
    assert open(tmp_path / "r.md").read().count("\n") == 2 + 5 and open(tmp_path / "r.csv").readline().startswith("kind,tp")


def test_convert_file_descriptors_exist_and_select_the_family():
    """Every `convert_file:` key of a model YAML points at a descriptor in the tree, and the converter reads it."""
    import glob
    import re

    from tools.convert_checkpoint import convert as C
    from tools.convert_checkpoint.name_maps import FAMILIES

    root = os.path.join(os.path.dirname(__file__), "..")
    seen = 0
    for y in glob.glob(os.path.join(root, "configs", "models", "**", "*.yaml"), recursive=True):
        for line in open(y):
            m = re.match(r"\s*convert_file:\s*\$\{oc\.env:LOONGFORGE_PATH\}/(\S+)", line)
            if m:
                path = os.path.join(root, m.group(1))
                assert os.path.isfile(path), f"{y} names {m.group(1)}, which does not exist"
                a = C.parse_args(["--load_platform", "huggingface", "--save_platform", "mcore", "--load_ckpt_path", "x",
                                  "--save_ckpt_path", "y", "--convert_file", path])
                assert a.model_type_custom in FAMILIES and a.safetensors
                seen += 1
    assert seen >= 4


@pytest.mark.parametrize("family,model", [("llama3", "tiny-llama"), ("qwen3_moe", "tiny-qwen3-moe")])
def test_hf_roundtrip_tool(tmp_path, family, model):
    from loongforge_b200.parallel import state as ps
    from tools.dist_checkpoint import hf_roundtrip as R

    ps.destroy_model_parallel()
    try:
        rep_path = tmp_path / "rep.json"
        assert R.main(["--synthetic", "--family", family, "--model-name", model, "--work-dir", str(tmp_path / "w"),
                       "--report", str(rep_path)]) == 0
        rep = json.load(open(rep_path))
        assert rep["ok"] and rep["compared"] > 5 and rep["tensors_exported"] == rep["compared"]
        # a corrupted tensor is reported
        import torch
        a = {"x": torch.ones(2), "y": torch.zeros(3)}
        bad = R.compare_state_dicts(a, {"x": torch.ones(2) * 2, "z": torch.zeros(1)})
        assert not bad["ok"] and bad["missing_in_result"] == ["y"] and bad["extra_in_result"] == ["z"]
        assert bad["value_mismatch"][0]["max_abs_diff"] == 1.0
    finally:
        ps.destroy_model_parallel()


def test_vlm_offline_packing_pipeline_and_loader(tmp_path):
    """scan -> plan -> write over image-text shards, then the loader keeps every offline pack together."""
    import numpy as np

    from loongforge_b200.data.multimodal import VisionPreprocess, is_packed_dataset, vlm_batch_iterator, webdataset_samples
    from loongforge_b200.data.task_encoders import SpecialTokens, build_task_encoder
    from tools.data_preprocess import vlm_offline_packing as P
    from tools.data_preprocess.vlm_to_webdataset import write_shards

    rng = np.random.RandomState(0)
    img_dir = tmp_path / "img"
    img_dir.mkdir()
    recs = []
    for i in range(12):
        h, w = int(rng.choice([28, 56, 84])), int(rng.choice([28, 56]))
        np.save(img_dir / f"{i}.npy", rng.randint(0, 255, (h, w, 3), dtype=np.uint8))
        recs.append({"image": f"{i}.npy", "conversations": [{"from": "human", "value": "<image> " + "word " * int(rng.randint(2, 30))},
                                                            {"from": "gpt", "value": "ok " * int(rng.randint(1, 10))}]})
    write_shards(recs, str(tmp_path / "src"), str(img_dir), samples_per_shard=5)
    out = P.main(["all", "--shards", str(tmp_path / "src"), "--output-dir", str(tmp_path / "dst"), "--seq-length", "128",
                  "--packs-per-shard", "2", "--min-pixels", "784", "--max-pixels", "50176"])
    assert out["scanned"] == 12 and out["plan"]["dropped"] == 0 and 0.3 < out["plan"]["fill_rate"] <= 1.0
    assert P.scan(str(tmp_path / "src"), str(tmp_path / "dst" / "manifest.sqlite")) == 0  # resumable: nothing left
    assert is_packed_dataset(str(tmp_path / "dst")) and not is_packed_dataset(str(tmp_path / "src"))
    idx = json.load(open(tmp_path / "dst" / "index.json"))
    assert idx["total"] == 12 and idx["packs"] == out["plan"]["packs"] and len(idx["shards"]) == -(-idx["packs"] // 2)
    # every rank sees whole packs; together the ranks see every sample once
    seen = []
    for r in range(2):
        got = list(webdataset_samples(str(tmp_path / "dst"), dp_rank=r, dp_size=2, epochs=1))
        by_pack = {}
        for s in got:
            by_pack.setdefault(s["pack_id"], []).append(s)
        assert all(len(v) == v[0]["pack_size"] for v in by_pack.values())
        seen += got
    assert len(seen) == 12
    enc = build_task_encoder("qwen2_vl", lambda t: [10 + (ord(c) % 50) for c in t], SpecialTokens(image=900, eos=2),
                             VisionPreprocess(min_pixels=784, max_pixels=50176))
    rows = list(vlm_batch_iterator(webdataset_samples(str(tmp_path / "dst"), epochs=1), enc, 512))
    assert len(rows) == idx["packs"] and all(b["tokens"].shape == (1, 512) for b in rows)
    assert sum(b["grid_thw"].shape[0] for b in rows) == 12


def test_pretrain_preprocessing_partitions_sentences_and_resume(tmp_path):
    """Partitioned runs merge to the same data set as one pass (round-robin and sequential dealing); sentence splitting
    keeps document boundaries; gzip input and globs; a finished partition is not redone."""
    import gzip
    import json as js
    import numpy as np
    from loongforge_b200.data.indexed_dataset import IndexedDataset
    from tools.data_preprocess import preprocess_pretrain_data as pp

    docs = [{"text": f"Document {i} starts here. It has a second sentence! And a third one?\nNew line {i}.", "title": f"t{i}"}
            for i in range(11)]
    (tmp_path / "a.jsonl").write_text("\n".join(js.dumps(d) for d in docs[:6]) + "\n")
    with gzip.open(tmp_path / "b.jsonl.gz", "wt") as f:
        f.write("\n".join(js.dumps(d) for d in docs[6:]) + "\n")
    glob_in = str(tmp_path / "*.jsonl*")
    pp.main(["--input", glob_in, "--output-prefix", str(tmp_path / "one" / "c"), "--append-eod", "--json-keys", "text", "title"])
    one = IndexedDataset(str(tmp_path / "one" / "c_text_document"))
    assert len(one) == 11 and len(IndexedDataset(str(tmp_path / "one" / "c_title_document"))) == 11
    pp.main(["--input", glob_in, "--output-prefix", str(tmp_path / "seq" / "c"), "--append-eod", "--partitions", "3",
             "--keep-sequential-samples", "--workers", "2"])
    seq = IndexedDataset(str(tmp_path / "seq" / "c_text_document"))
    assert len(seq) == 11 and all(np.array_equal(seq[i], one[i]) for i in range(11))          # contiguous ranges: same order
    assert list(seq.doc_idx) == list(range(12)) and not any("part" in f for f in os.listdir(tmp_path / "seq"))
    pp.main(["--input", glob_in, "--output-prefix", str(tmp_path / "rr" / "c"), "--append-eod", "--partitions", "3"])
    rr = IndexedDataset(str(tmp_path / "rr" / "c_text_document"))
    assert sorted(bytes(rr[i]) for i in range(11)) == sorted(bytes(one[i]) for i in range(11))  # round-robin: same documents
    pp.main(["--input", glob_in, "--output-prefix", str(tmp_path / "sent" / "c"), "--append-eod", "--split-sentences", "--keep-newlines"])
    sent = IndexedDataset(str(tmp_path / "sent" / "c_text_sentence"))
    assert len(sent) == 44 and list(sent.doc_idx) == list(range(0, 45, 4))                     # four sentences per document
    assert sent[3][-1] == 257 and sent[2][-1] != 257                                          # end-of-document on the last one
    assert sent.num_tokens == one.num_tokens - 11 * 3            # separators (3 per document) are not tokens of any sentence
    assert pp.split_sentences("A b. C d! E\nF", keep_newlines=False) == ["A b.", "C d!", "E F"]


def test_sft_preprocessing_masks_splits_packing_and_trainer_reads_shards(tmp_path):
    from loongforge_b200.data.sft import SFTDataset
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer
    from tools.data_preprocess import preprocess_sft_data as P

    assert P.mask_history([-100, 5, 6, -100, -100, 7, 8, -100]) == [-100, -100, -100, -100, -100, 7, 8, -100]
    assert P.mask_run_ends([-100, 5, 6, -100, 7]) == [-100, 5, -100, -100, -100]
    recs = [{"messages": [{"role": "user", "content": f"q{i} " + "a" * (7 * i)}, {"role": "assistant", "content": "first"},
                          {"role": "user", "content": "again"}, {"role": "assistant", "content": "second answer"}]} for i in range(20)]
    src = tmp_path / "chat.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in recs))
    out = tmp_path / "o"
    P.main(["--input", str(src), "--output-path", str(out), "--seq-length", "4096", "--split", "80,10,10", "--history-mask-loss",
            "--context-parallel-size", "2", "--sft-sort-batch", "--workers", "2"])
    idx = json.load(open(out / "index.json"))
    assert {k: v["num_samples"] for k, v in idx["splits"].items()} == {"train": 16, "valid": 2, "test": 2}
    rows = [json.loads(l) for l in open(out / "train_00000.jsonl")]
    lens = [len(r["input_ids"]) for r in rows]
    assert lens == sorted(lens) and all(n % 4 == 0 for n in lens)                  # sorted, padded to 2 x cp
    tok = build_tokenizer("ByteTokenizer")
    tgt = bytes(t for t in rows[0]["labels"] if t != -100 and t < 256).decode()
    assert "second answer" in tgt and "first" not in tgt                             # only the last turn is trained
    plain = tmp_path / "p"
    P.main(["--input", str(src), "--output-path", str(plain), "--seq-length", "4096"])
    both = bytes(t for t in json.loads(open(plain / "train_00000.jsonl").readline())["labels"] if t != -100 and t < 256).decode()
    assert "first" in both and "second answer" in both
    packed = tmp_path / "k"
    P.main(["--input", str(src), "--output-path", str(packed), "--seq-length", "600", "--packing-sft-data", "--packing-buffer-size", "4"])
    prow = [json.loads(l) for l in open(packed / "train_00000.jsonl")]
    assert len(prow) < 20 and all(len(r["input_ids"]) <= 600 and sum(r["seq_lens"]) == len(r["input_ids"]) for r in prow)
    assert sum(len(r["seq_lens"]) for r in prow) == 20
    # the trainer's data set takes the shard as it is
    ds = SFTDataset([str(plain / "train_00000.jsonl")], tok, max_len=4096)
    ids, labels = ds[3]
    ref = json.loads(open(plain / "train_00000.jsonl").readlines()[3])
    assert ids == ref["input_ids"] and labels == ref["labels"]


def test_every_conversion_descriptor_names_a_known_family():
    import glob
    from types import SimpleNamespace as NS
    from tools.convert_checkpoint import convert as C
    from tools.convert_checkpoint.name_maps import FAMILIES

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "configs", "models", "*", "ckpt_convert", "*.yaml")))
    assert len(files) >= 18
    for f in files:
        a = NS(model_type_custom="llama3", safetensors=False, make_vocab_size_divisible_by=128)
        C.apply_convert_file(a, f)
        assert a.model_type_custom in FAMILIES, (f, a.model_type_custom)
        assert a.safetensors is True
    a = NS(model_type_custom="llama3", safetensors=False, make_vocab_size_divisible_by=128)
    C.apply_convert_file(a, os.path.join(root, "configs/models/kimi_k2/ckpt_convert/kimi_k2_convert.yaml"))
    assert a.model_type_custom == "kimi_k2" and a.make_vocab_size_divisible_by == 1280


def test_compare_checkpoints_tool(tmp_path, capsys):
    from safetensors.torch import save_file
    from tools.dist_checkpoint import compare_checkpoints as CC

    torch.manual_seed(0)
    a = {"w": torch.randn(4, 4), "b": torch.randn(4), "only_a": torch.zeros(1), "s": torch.randn(2, 3)}
    b = {"w": a["w"].clone(), "b": a["b"] + 1e-3, "only_b": torch.zeros(1), "s": torch.randn(3, 2)}
    os.makedirs(tmp_path / "A")
    os.makedirs(tmp_path / "B")
    save_file(a, str(tmp_path / "A" / "model.safetensors"))
    torch.save(b, tmp_path / "B" / "pytorch_model.bin")
    rc = CC.main([str(tmp_path / "A"), str(tmp_path / "B"), "--report", str(tmp_path / "r.json")])
    rep = json.load(open(tmp_path / "r.json"))
    assert rc == 1 and rep["only_in_a"] == ["only_a"] and rep["only_in_b"] == ["only_b"] and rep["matched"] == 1
    assert rep["shape_mismatch"][0]["key"] == "s" and rep["value_mismatch"][0]["key"] == "b" and abs(rep["max_abs_diff"] - 1e-3) < 1e-5
    out = capsys.readouterr().out
    assert "DIFFERENT" in out and "only in A: 1 (only_a)" in out and "value  b:" in out
    assert CC.main([str(tmp_path / "A"), str(tmp_path / "B"), "--atol", "1e-2", "--ignore", "^only_", "^s$"]) == 0
    assert CC.main([str(tmp_path / "A" / "model.safetensors"), str(tmp_path / "A")]) == 0
