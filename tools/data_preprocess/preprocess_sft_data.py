"""Offline tokenisation of SFT conversations: alpaca / sharegpt / openai-messages records -> token ids + labels
(prompt positions masked) with a chat template, written as JSONL shards with a length index for the packers
(reference: tools/data_preprocess SFT pre-tokenise)."""
from __future__ import annotations

import argparse
import json
import os
from typing import Iterable, List


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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--tokenizer", default="null", help="'null' (byte-level) or a Hugging Face tokenizer directory")
    ap.add_argument("--chat-template", default="chatml")
    ap.add_argument("--format", default="auto", choices=["auto", "alpaca", "sharegpt", "openai"])
    ap.add_argument("--max-length", type=int, default=4096)
    ap.add_argument("--shard-size", type=int, default=100000)
    args = ap.parse_args(argv)

    from loongforge_b200.data.chat_template import encode_chat, to_messages
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer

    tok = build_tokenizer("ByteTokenizer") if args.tokenizer == "null" else build_tokenizer("HFTokenizer", args.tokenizer)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_prefix)), exist_ok=True)
    lengths: List[int] = []
    shard, n_in_shard, out = 0, 0, None
    kept = dropped = 0
    for rec in iter_records(args.input):
        ids, labels = encode_chat(tok, to_messages(rec, args.format), args.chat_template)
        if len(ids) > args.max_length:
            dropped += 1
            continue
        if out is None or n_in_shard >= args.shard_size:
            if out is not None:
                out.close()
            out = open(f"{args.output_prefix}_{shard:05d}.jsonl", "w")
            shard, n_in_shard = shard + 1, 0
        out.write(json.dumps({"input_ids": ids, "labels": labels}) + "\n")
        lengths.append(len(ids))
        n_in_shard += 1
        kept += 1
    if out is not None:
        out.close()
    with open(f"{args.output_prefix}_index.json", "w") as f:
        json.dump({"num_samples": kept, "dropped_too_long": dropped, "shards": shard, "lengths": lengths}, f)
    return kept, dropped


if __name__ == "__main__":
    main()
