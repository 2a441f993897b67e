"""Offline tokenisation of SFT conversations: alpaca / sharegpt / openai-messages records -> token ids + labels (prompt
positions masked) with a chat template, written as JSONL shards per split with a length index; the trainer reads the
shards through ``--sft-dataset <shard>`` without tokenising again (reference:
tools/data_preprocess/llm/preprocess_sft_data.py:78-225).

    python -m tools.data_preprocess.preprocess_sft_data --input chats.jsonl --output-path out/ --chat-template qwen \\
        --hf-tokenizer-path <dir> --seq-length 4096 --split 98,2,0 --workers 8 [--packing-sft-data]

* ``--split a,b,c``            train / valid / test shares (deterministic by record index);
* ``--train-on-prompt``        prompts are targets too; ``--history-mask-loss``: only the LAST assistant turn is a target;
  ``--eod-mask-loss``: the end-of-turn / end-of-document token at the end of a target run is not a target;
* ``--enable-discard-sample``  samples longer than ``--seq-length`` are dropped (default: truncated);
* ``--context-parallel-size``  sample lengths are padded (token 0, label -100) to a multiple of ``2 x cp``;
* ``--sft-sort-batch``         samples of a split are written in order of length (fewer padded tokens per batch);
* ``--packing-sft-data``       samples are packed offline into rows of at most ``--seq-length`` tokens (first-fit over a
  buffer of ``--packing-buffer-size`` samples); a packed record also carries ``seq_lens``.
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import sys
from typing import Iterable, List, Optional, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_STATE = {}


def iter_records(path: str) -> Iterable[dict]:
    with open(path) as f:
        head = f.read(1)
        f.seek(0)
        if head == "[":
            yield from json.load(f)
        else:
            for line in f:
                if line.strip():
                    yield json.loads(line)


def _init(tok_type, tok_path, template, fmt, opts):
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer
    _STATE["tok"] = build_tokenizer(tok_type, tok_path) if tok_type != "ByteTokenizer" else build_tokenizer("ByteTokenizer")
    _STATE.update(template=template, fmt=fmt, **opts)


def mask_history(labels: List[int]) -> List[int]:
    """Keeps the last run of target positions, masks the earlier ones."""
    end = len(labels)
    while end > 0 and labels[end - 1] == -100:
        end -= 1
    start = end
    while start > 0 and labels[start - 1] != -100:
        start -= 1
    return [-100] * start + labels[start:end] + [-100] * (len(labels) - end)


def mask_run_ends(labels: List[int]) -> List[int]:
    out = list(labels)
    for i, v in enumerate(labels):
        if v != -100 and (i + 1 == len(labels) or labels[i + 1] == -100):
            out[i] = -100
    return out


def _encode(rec: dict) -> Optional[Tuple[List[int], List[int]]]:
    from loongforge_b200.data.chat_template import encode_chat, to_messages
    s = _STATE
    ids, labels = encode_chat(s["tok"], to_messages(rec, s["fmt"]), s["template"], s["train_on_prompt"], tools=rec.get("tools"))
    if s["history_mask_loss"]:
        labels = mask_history(labels)
    if s["eod_mask_loss"]:
        labels = mask_run_ends(labels)
    L = s["seq_length"]
    if L and len(ids) > L:
        if s["discard"]:
            return None
        ids, labels = ids[:L], labels[:L]
    m = 2 * s["cp"]
    if m > 1 and len(ids) % m:
        pad = m - len(ids) % m
        ids, labels = ids + [0] * pad, labels + [-100] * pad
    if all(v == -100 for v in labels):
        return None
    return ids, labels


def pack_first_fit(samples: List[Tuple[List[int], List[int]]], seq_length: int, buffer_size: int) -> List[dict]:
    rows: List[dict] = []
    open_rows: List[dict] = []
    for ids, labels in samples:
        for r in open_rows:
            if len(r["input_ids"]) + len(ids) <= seq_length:
                r["input_ids"] += ids
                r["labels"] += labels
                r["seq_lens"].append(len(ids))
                break
        else:
            open_rows.append({"input_ids": list(ids), "labels": list(labels), "seq_lens": [len(ids)]})
            if len(open_rows) > buffer_size:
                rows.append(open_rows.pop(0))
    return rows + open_rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output-path", "--output-prefix", dest="output_path", required=True)
    ap.add_argument("--seq-length", "--max-length", dest="seq_length", type=int, default=4096)
    ap.add_argument("--split", default="100,0,0")
    ap.add_argument("--context-parallel-size", type=int, default=1)
    ap.add_argument("--tokenizer-type", default=None)
    ap.add_argument("--hf-tokenizer-path", "--tokenizer", dest="hf_tokenizer_path", default=None,
                    help="Hugging Face tokenizer directory ('null' or nothing: byte-level tokenizer)")
    ap.add_argument("--use-fast-tokenizer", action="store_true")
    ap.add_argument("--split-special-tokens", action="store_true")
    ap.add_argument("--additional-special-tokens", default=None)
    ap.add_argument("--chat-template", default="chatml")
    ap.add_argument("--chat-template-kwargs", default=None)
    ap.add_argument("--sft-dataset-config", default=None)
    ap.add_argument("--sft-dataset", "--format", dest="fmt", default="auto")
    ap.add_argument("--packing-sft-data", action="store_true")
    ap.add_argument("--packing-buffer-size", type=int, default=1000)
    ap.add_argument("--sft-sort-batch", action="store_true")
    ap.add_argument("--image-resolution", type=int, default=None)
    ap.add_argument("--train-on-prompt", action="store_true")
    ap.add_argument("--history-mask-loss", action="store_true")
    ap.add_argument("--eod-mask-loss", action="store_true")
    ap.add_argument("--enable-discard-sample", action="store_true")
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--shard-size", type=int, default=100000)
    a = ap.parse_args(argv)

    byte_level = a.hf_tokenizer_path in (None, "null")
    tok_type = "ByteTokenizer" if byte_level else (a.tokenizer_type or "HFTokenizer")
    fmt = a.fmt if a.fmt in ("auto", "alpaca", "sharegpt", "openai") else "auto"
    opts = dict(train_on_prompt=a.train_on_prompt, history_mask_loss=a.history_mask_loss, eod_mask_loss=a.eod_mask_loss,
                seq_length=a.seq_length, discard=a.enable_discard_sample, cp=a.context_parallel_size)
    init = (tok_type, None if byte_level else a.hf_tokenizer_path, a.chat_template, fmt, opts)
    records = list(iter_records(a.input))
    if a.workers > 1:
        with mp.Pool(a.workers, initializer=_init, initargs=init) as pool:
            encoded = pool.map(_encode, records, chunksize=64)
    else:
        _init(*init)
        encoded = [_encode(r) for r in records]
    shares = [float(x) for x in a.split.split(",")] + [0.0, 0.0]
    total = sum(shares[:3]) or 1.0
    bounds = [shares[0] / total, (shares[0] + shares[1]) / total]
    splits = {"train": [], "valid": [], "test": []}
    dropped = 0
    n = max(len(encoded), 1)
    for i, e in enumerate(encoded):
        if e is None:
            dropped += 1
            continue
        frac = (i + 0.5) / n
        splits["train" if frac <= bounds[0] else "valid" if frac <= bounds[1] else "test"].append(e)
    os.makedirs(a.output_path if not a.output_path.endswith(".jsonl") else os.path.dirname(a.output_path) or ".", exist_ok=True)
    summary = {"dropped": dropped, "splits": {}}
    for name, samples in splits.items():
        if not samples:
            continue
        if a.sft_sort_batch:
            samples = sorted(samples, key=lambda s: len(s[0]))
        rows = (pack_first_fit(samples, a.seq_length, a.packing_buffer_size) if a.packing_sft_data
                else [{"input_ids": i, "labels": l} for i, l in samples])
        files, lengths = [], []
        for shard in range(0, len(rows), a.shard_size):
            path = os.path.join(a.output_path, f"{name}_{shard // a.shard_size:05d}.jsonl")
            with open(path, "w") as f:
                for r in rows[shard:shard + a.shard_size]:
                    f.write(json.dumps(r) + "\n")
                    lengths.append(len(r["input_ids"]))
            files.append(os.path.basename(path))
        summary["splits"][name] = {"num_samples": len(samples), "num_rows": len(rows), "shards": files, "lengths": lengths,
                                   "tokens": sum(lengths), "packed": bool(a.packing_sft_data)}
    with open(os.path.join(a.output_path, "index.json"), "w") as f:
        json.dump(summary, f)
    kept = sum(v["num_samples"] for v in summary["splits"].values())
    print(json.dumps({"kept": kept, "dropped": dropped, **{k: v["num_rows"] for k, v in summary["splits"].items()}}))
    return kept, dropped


if __name__ == "__main__":
    main()
