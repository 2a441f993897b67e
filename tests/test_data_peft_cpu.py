"""Data pipeline (chat templates, packing, indexed datasets), tokenizer, LoRA and the VLM trainer on CPU."""
import json
import os

import numpy as np
import pytest
import torch


def test_chat_template_masks_only_assistant_tokens():
    from loongforge_b200.data.chat_template import encode_chat, to_messages
    from loongforge_b200.tokenizer.tokenizer import ByteTokenizer

    tok = ByteTokenizer(["<|im_start|>", "<|im_end|>"])
    msgs = to_messages({"instruction": "Add", "input": "1+1", "output": "2"})
    ids, labels = encode_chat(tok, msgs, "chatml")
    assert len(ids) == len(labels)
    tgt = [i for i, l in zip(ids, labels) if l != -100]
    assert tok.detokenize(tgt) == "2<|im_end|>\n"
    assert tok.detokenize(ids).startswith("<|im_start|>user\nAdd\n1+1<|im_end|>")
    sg = to_messages({"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "yo"}]})
    assert [m["role"] for m in sg] == ["user", "assistant"]


def test_packing_and_lpt():
    from loongforge_b200.data.packing import collate_packed, lpt_partition, pack_first_fit_decreasing

    lens = [900, 300, 700, 120, 60, 1000, 40]
    bins = pack_first_fit_decreasing(lens, 1024)
    assert sorted(i for b in bins for i in b) == list(range(len(lens)))
    assert all(sum(min(lens[i], 1024) for i in b) <= 1024 for b in bins)
    groups = lpt_partition([5, 3, 3, 2, 2, 1], 2)
    loads = [sum([5, 3, 3, 2, 2, 1][i] for i in g) for g in groups]
    assert abs(loads[0] - loads[1]) <= 1
    b = collate_packed([([1, 2, 3, 4], [-100, -100, 3, 4]), ([5, 6, 7], [-100, 6, 7])], 16)
    assert b["tokens"].shape == (1, 16) and b["cu_seqlens"].tolist() == [0, 4, 7, 16]
    assert b["position_ids"][0, :7].tolist() == [0, 1, 2, 3, 0, 1, 2]
    assert b["loss_mask"][0, :7].tolist() == [0, 1, 1, 0, 1, 1, 0] and b["num_valid_tokens"] == 4


def test_indexed_dataset_roundtrip(tmp_path):
    from loongforge_b200.data.indexed_dataset import GPTDataset, IndexedDataset, IndexedDatasetWriter

    w = IndexedDatasetWriter(str(tmp_path / "corpus"), np.int32)
    docs = [list(range(10)), list(range(100, 137)), [7, 8, 9, 1]]
    for d in docs:
        w.add_document(d)
    w.finalize()
    ds = IndexedDataset(str(tmp_path / "corpus"))
    assert len(ds) == 3 and [ds[i].tolist() for i in range(3)] == docs and ds.num_tokens == 51
    g = GPTDataset(ds, seq_length=8, num_samples=5, seed=1)
    s = g[0]
    assert s["tokens"].shape == (8,) and torch.equal(s["tokens"][1:], s["labels"][:-1])


def test_lora_trains_only_adapters_and_merges():
    from loongforge_b200.models.gpt import GPTModel
    from loongforge_b200.models.peft import adapter_state_dict, apply_lora, merge_lora
    from loongforge_b200.models.registry import get_model_config

    torch.manual_seed(0)
    m = GPTModel(get_model_config("tiny-llama"))
    T = 32
    tok = torch.randint(0, 32000, (T,))
    base = m(tok, torch.arange(T))
    names = apply_lora(m, rank=4, alpha=8, canonical=True)
    assert len(names) == 8
    assert torch.allclose(m(tok, torch.arange(T)), base, atol=1e-5)  # B starts at zero
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.02)
    tuned = m(tok, torch.arange(T))
    assert len(adapter_state_dict(m)) == 16
    assert merge_lora(m) == 8
    assert torch.allclose(m(tok, torch.arange(T)), tuned, atol=1e-4)


def test_sft_trainer_with_packed_data(tmp_path):
    from loongforge_b200.data.sft import SFTDataset, sft_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.runtime.sft import SFTTrainer
    from loongforge_b200.runtime.trainer import TrainConfig
    from loongforge_b200.tokenizer.tokenizer import ByteTokenizer

    p = tmp_path / "d.jsonl"
    with open(p, "w") as f:
        for i in range(40):
            f.write(json.dumps({"instruction": f"say {i}", "output": "ok " * (i % 7 + 1)}) + "\n")
    tok = ByteTokenizer(["<|im_start|>", "<|im_end|>"])
    ds = SFTDataset([str(p)], tok, max_len=128)
    it = sft_batch_iterator(ds, 128, packing=True, pad_id=tok.pad)
    cfg = get_model_config("tiny-llama", vocab_size=tok.vocab_size, make_vocab_size_divisible_by=8)
    tr = SFTTrainer(cfg, TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=128, train_iters=4, lr=2e-3,
                                     training_phase="sft", log_interval=100), lora=dict(rank=4, alpha=8))
    losses = [tr.train_step(it)["lm loss"] for _ in range(6)]
    assert losses[-1] < losses[0]


def test_vlm_trainer_loss_on_text_only():
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.runtime.trainer import TrainConfig
    from loongforge_b200.runtime.vlm import VLMTrainer, synthetic_vlm_iterator

    lm = get_model_config("tiny-llama", position_embedding_type="mrope", mrope_section=[8, 12, 12])
    vit = get_model_config("tiny-vit")
    tr = VLMTrainer(lm, TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=128, train_iters=2, lr=1e-3,
                                    log_interval=100), vit_cfg=vit)
    it = synthetic_vlm_iterator(lm.vocab_size, 128, images_per_sample=2, image_size=112, pin_memory=False)
    b = next(it)
    assert b["pixels"].shape == (2 * 64, 3 * 2 * 14 * 14) and (b["tokens"] == lm.vocab_size - 1).sum() == 2 * 16
    assert float((b["loss_mask"][0][b["tokens"][0] == lm.vocab_size - 1]).sum()) == 0.0
    m = tr.train_step(it)
    assert np.isfinite(m["lm loss"]) and m["grad_norm"] > 0


def test_internvl_tiling_and_ernie_positions():
    import torch
    from loongforge_b200.runtime import sft_families as F

    assert F.internvl_tile_grid(448, 448) == (1, 1)
    assert F.internvl_tile_grid(1792, 448, max_tiles=6) == (4, 1)
    assert F.internvl_tile_grid(896, 1344, max_tiles=6) == (2, 3)
    assert F.internvl_num_tiles(448, 448) == 1 and F.internvl_num_tiles(896, 1344, max_tiles=6) == 7
    ids, tiles = F.internvl_expand_image_tokens([1, 9, 2], [(896, 448)], image_marker_id=9, img_start_id=5,
                                                img_context_id=6, img_end_id=7, tokens_per_tile=4, max_tiles=4)
    assert tiles == [3] and ids == [1, 5] + [6] * 12 + [7, 2]
    b = F.internvl_batch([{"input_ids": [1, 2, 3], "labels": [-100, 2, 3], "pixel_tiles": torch.zeros(2, 3, 448, 448)},
                          {"input_ids": [4, 5], "labels": [-100, 5], "pixel_tiles": None}])
    assert b["cu_seqlens"].tolist() == [0, 3, 5] and b["loss_mask"].tolist() == [1, 1, 0, 1, 0]
    assert b["pixel_tiles"].shape[0] == 2
    tok = torch.tensor([3, 4, 8, 8, 8, 8, 8, 8, 5])
    tt, pos = F.ernie_token_types_and_positions(tok, 8, [(2, 3)])
    assert tt.tolist() == [0, 0, 1, 1, 1, 1, 1, 1, 0]
    assert pos[0].tolist() == [0, 1, 2, 2, 2, 2, 2, 2, 5]
    assert pos[1].tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 5] and pos[2].tolist() == [0, 1, 2, 3, 4, 2, 3, 4, 5]


def test_pretrain_data_path_split_blend_and_evaluation(tmp_path):
    """--data-path (weighted blend of two .bin/.idx prefixes) + --split + --eval-interval through the CLI."""
    import re
    import subprocess
    import sys

    from loongforge_b200.data import indexed_dataset as I

    rng = np.random.RandomState(0)
    for name, lo in (("a", 0), ("b", 500)):
        w = I.IndexedDatasetWriter(str(tmp_path / name))
        for _ in range(40):
            w.add_document(list(rng.randint(lo, lo + 400, size=rng.randint(50, 200))) + [999])
        w.finalize()
    assert I.split_document_ranges(40, "949,50,1") == [(0, 38), (38, 40), (40, 40)]
    assert I.parse_data_path(["0.25", "x", "0.75", "y"]) == ([0.25, 0.75], ["x", "y"])
    tr, va, te = I.build_gpt_datasets(["0.25", str(tmp_path / "a"), "0.75", str(tmp_path / "b")], "90,10,0", 32,
                                      (64, 8, 0))
    assert te is None and len(tr) == 64 and len(va) == 8
    from_b = sum(int(tr[i]["tokens"].max() >= 500) for i in range(64))
    assert 44 <= from_b <= 52, "three quarters of the stream come from the second prefix"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "loongforge_b200.train", "--model-name", "tiny-llama", "--vocab-size", "1024",
           "--seq-length", "32", "--micro-batch-size", "2", "--global-batch-size", "4", "--train-iters", "4",
           "--lr", "1e-3", "--log-interval", "1", "--data-path", "0.25", str(tmp_path / "a"), "0.75", str(tmp_path / "b"),
           "--split", "90,10,0", "--eval-interval", "2", "--eval-iters", "1"]
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert p.returncode == 0, p.stderr[-2000:]
    evals = re.findall(r"validation loss at iteration (\d+) \| lm loss value: ([0-9.E+-]+) \| lm loss PPL: ([0-9.E+-]+)",
                       p.stdout)
    assert [int(e[0]) for e in evals] == [2, 4] and all(float(e[1]) < 8.0 for e in evals)


def test_vlm_lora_per_component():
    """Adapters on chosen components of a vision-language model: the language model alone (default), the vision tower
    and projector as well; a component that is frozen cannot also get adapters."""
    import pytest
    import torch

    from loongforge_b200.models.omni import OmniCombinationModel
    from loongforge_b200.models.peft import apply_vlm_lora
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    try:
        def build():
            lm = get_model_config("tiny-llama", position_embedding_type="mrope", mrope_section=[8, 12, 12])
            return OmniCombinationModel(lm, get_model_config("tiny-vit"), image_token_id=lm.vocab_size - 1)

        def trainable(m):
            return {n for n, p in m.named_parameters() if p.requires_grad}

        m = build()
        w = apply_vlm_lora(m, rank=2, alpha=4)
        t = trainable(m)
        assert set(w) == {"foundation"} and w["foundation"]
        assert all("lora_" in n for n in t if n.startswith("foundation_model."))
        assert any(n.startswith("encoder_model.image_encoder.") for n in t)  # untouched component keeps training

        m = build()
        w = apply_vlm_lora(m, rank=2, alpha=4, apply_to_image_encoder=True, apply_to_image_projector=True)
        t = trainable(m)
        assert set(w) == {"foundation", "image_encoder", "image_projector"} and w["image_encoder"]
        assert all("lora_" in n for n in t), sorted(t)[:5]

        m = build()
        apply_vlm_lora(m, rank=2, alpha=4, apply_to_foundation=False, apply_to_image_encoder=True, frozen=("image_projector",))
        t = trainable(m)
        assert not any(n.startswith("encoder_model.image_projector.") for n in t)
        assert any(n.startswith("foundation_model.") and "lora_" not in n for n in t)
        with pytest.raises(ValueError, match="cannot freeze"):
            apply_vlm_lora(build(), rank=2, apply_to_image_encoder=True, frozen=("image_encoder",))
    finally:
        ps.destroy_model_parallel()


def test_named_sft_dataset_layouts(tmp_path):
    """--sft-dataset as layout names (the reference's launchers): columns and tags of configs/data/sft_dataset_config.yaml
    map alpaca records with history, renamed sharegpt keys, openai tools and function calls to chat messages."""
    import json
    from types import SimpleNamespace as NS
    from loongforge_b200.data import sft_formats as F
    from loongforge_b200.data.sft import SFTDataset
    from loongforge_b200.runtime.sft import sft_paths_and_formats
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer

    table = F.load_dataset_config()
    assert {"default", "alpaca", "extended_alpaca", "sharegpt", "openai", "multimodal", "multimodal_sharegpt"} <= set(table)
    m, tools, _ = F.convert({"instruction": "Add", "input": "1 2", "output": "3", "system": "calc", "history": [["hi", "hello"]]},
                            table["extended_alpaca"])
    assert [x["role"] for x in m] == ["system", "user", "assistant", "user", "assistant"] and m[3]["content"] == "Add\n1 2"
    m, _, imgs = F.convert({"messages": [{"from": "human", "value": "<image> what"}, {"from": "gpt", "value": "a cat"}], "images": ["a.jpg"]},
                           table["multimodal_sharegpt"])
    assert [x["role"] for x in m] == ["user", "assistant"] and imgs == ["a.jpg"]
    rec = {"conversations": [{"from": "human", "value": "weather?"}, {"from": "function_call", "value": json.dumps({"name": "get", "arguments": {"c": "x"}})},
                             {"from": "observation", "value": "sunny"}, {"from": "gpt", "value": "It is sunny."}],
           "tools": json.dumps([{"name": "get"}]), "system": "be brief"}
    m, tools, _ = F.convert(rec, table["sharegpt_conversations"])
    assert [x["role"] for x in m] == ["system", "user", "assistant", "tool", "assistant"]
    assert m[2]["tool_calls"][0]["function"]["name"] == "get" and tools == [{"name": "get"}]
    with pytest.raises(ValueError):
        F.convert({"messages": [{"role": "narrator", "content": "x"}]}, table["openai"])
    with pytest.raises(KeyError):
        F.resolve_formats(["nope"], 1)
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text(json.dumps({"instruction": "say hi", "input": "", "output": "hi"}) + "\n")
    b.write_text(json.dumps({"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "ans"}]}) + "\n")
    args = NS(sft_dataset=["alpaca", "openai"], data_path=[str(a), str(b)], train_data_path=None, sft_train_dataset=None, sft_dataset_config=None)
    paths, fmts = sft_paths_and_formats(args)
    assert paths == [str(a), str(b)] and [f.name for f in fmts] == ["alpaca", "openai"]
    ds = SFTDataset(paths, build_tokenizer("ByteTokenizer"), formats=fmts)
    texts = [bytes(t for t in ds[i][1] if t != -100 and t < 256).decode() for i in range(2)]
    assert any("hi" in t for t in texts) and any("ans" in t for t in texts)
    assert sft_paths_and_formats(NS(sft_dataset=[str(a)], data_path=None, train_data_path=None))[1] is None   # files as before
    with pytest.raises(ValueError):
        sft_paths_and_formats(NS(sft_dataset=["alpaca"], data_path=None, train_data_path=None, sft_train_dataset=None, sft_dataset_config=None))
    custom = tmp_path / "cfg.yaml"
    custom.write_text("mine:\n  format: alpaca\n  columns: {prompt: q, response: a}\n")
    m, _, _ = F.convert({"q": "Q?", "a": "A."}, F.load_dataset_config(str(custom))["mine"])
    assert m[0]["content"] == "Q?" and m[1]["content"] == "A."


def test_streaming_sft_iterator_and_mix_strategies(tmp_path):
    import json
    from loongforge_b200.data.sft import mixed_record_stream, streaming_sft_batch_iterator
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer

    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text("\n".join(json.dumps({"instruction": f"a{i}", "output": "x" * 10}) for i in range(5)) + "\n")
    b.write_text("\n".join(json.dumps({"instruction": f"b{i}", "output": "y" * 10}) for i in range(2)) + "\n")
    tag = lambda it: [r["instruction"] for r in it]  # noqa: E731
    assert tag(mixed_record_stream([str(a), str(b)], "concat")) == ["a0", "a1", "a2", "a3", "a4", "b0", "b1"]
    assert tag(mixed_record_stream([str(a), str(b)], "interleave_under")) == ["a0", "b0", "a1", "b1", "a2"]
    over = tag(mixed_record_stream([str(a), str(b)], "interleave_over"))
    assert over[:6] == ["a0", "b0", "a1", "b1", "a2", "b0"] and over.count("a4") == 1 and sum(x.startswith("a") for x in over) == 5
    tok = build_tokenizer("ByteTokenizer")
    seen = []
    for rank in range(2):
        it = streaming_sft_batch_iterator([str(a), str(b)], tok, 128, buffer_size=3, strategy="concat", dp_rank=rank, dp_size=2, seed=3)
        rows = []
        for _ in range(40):
            batch = next(it)
            rows.append(batch)
            text = bytes(t for t in batch["tokens"].flatten().tolist() if 0 < t < 256).decode()
            seen += [w for w in ("a0", "a1", "a2", "a3", "a4", "b0", "b1") if w in text]
            if len(set(seen)) == 7 and rank == 1:
                break
        assert rows[0]["tokens"].shape == (1, 128)
    assert set(seen) == {"a0", "a1", "a2", "a3", "a4", "b0", "b1"}            # every record reaches some rank
    it1 = streaming_sft_batch_iterator([str(a)], tok, 64, buffer_size=2, seed=5)
    it2 = streaming_sft_batch_iterator([str(a)], tok, 64, buffer_size=2, seed=5, start_sample=2)
    first = [next(it1) for _ in range(4)]
    assert torch.equal(next(it2)["tokens"], first[2]["tokens"])               # resuming skips what was consumed


def test_prefetch_iterator_order_errors_and_close():
    import time
    from loongforge_b200.data.samplers import PrefetchIterator

    def gen(n, fail_at=None):
        for i in range(n):
            if i == fail_at:
                raise RuntimeError("boom")
            time.sleep(0.002)
            yield i

    assert list(PrefetchIterator(gen(20), depth=3)) == list(range(20))
    it = PrefetchIterator(gen(10, fail_at=4), depth=2)
    got = []
    with pytest.raises(RuntimeError, match="boom"):
        for x in it:
            got.append(x)
    assert got == [0, 1, 2, 3]                                      # the error arrives at its position
    slow = PrefetchIterator(gen(10 ** 6), depth=2)
    assert next(slow) == 0
    t0 = time.perf_counter()
    slow.close()
    assert time.perf_counter() - t0 < 3 and not slow.thread.is_alive()
    # work overlaps: while the consumer sleeps the producer fills the queue
    p = PrefetchIterator(gen(8), depth=8)
    time.sleep(0.1)
    t0 = time.perf_counter()
    assert [next(p) for _ in range(8)] == list(range(8)) and time.perf_counter() - t0 < 0.01
