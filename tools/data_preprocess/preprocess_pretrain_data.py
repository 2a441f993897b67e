"""jsonl -> Megatron ``.bin`` / ``.idx`` pre-training data. Same role and flags as the reference's
tools/data_preprocess/llm/preprocess_pretrain_data.py.

    python -m tools.data_preprocess.preprocess_pretrain_data --input 'corpus/*.jsonl.gz' --output-prefix out/corpus \\
        --tokenizer-type HFTokenizer --hf-tokenizer-path <dir> --append-eod --workers 8 [--partitions 4]

* ``--input`` is a file or a glob; ``.gz`` files are read compressed; one JSON document per line, the text under each of
  ``--json-keys`` (one output data set per key: ``<prefix>_<key>_document.{bin,idx}``);
* ``--split-sentences``: a document becomes several items (one per sentence, ``--keep-newlines`` keeps line breaks as
  boundaries), the document index still marks documents (``<prefix>_<key>_sentence``);
* ``--partitions N``: the input lines are dealt to N partitions, each tokenised into files of its own by ``--workers``
  processes, then merged in order — a partition that already has its ``.idx`` is not redone, so an interrupted run
  resumes; ``--keep-sequential-samples`` deals contiguous ranges instead of round-robin;
* ``--append-eod`` appends the end-of-document token to every document (to its last sentence when split).
"""
from __future__ import annotations

import argparse
import glob
import gzip
import json
import multiprocessing as mp
import os
import re
import sys
import time
from typing import Iterator, List

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_TOK = None
_SENT = re.compile(r"(?<=[.!?。！？])\s+")


def _init(tok_type, path):
    global _TOK
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer
    _TOK = build_tokenizer(tok_type, path)


def split_sentences(text: str, keep_newlines: bool = False) -> List[str]:
    parts: List[str] = []
    for block in (text.split("\n") if keep_newlines else [text.replace("\n", " ")]):
        parts += [s for s in _SENT.split(block.strip()) if s]
    return parts


def _encode(args):
    line, keys, eod, split, keep_nl = args
    try:
        rec = json.loads(line)
    except json.JSONDecodeError:
        return {}, len(line)
    out = {}
    for k in keys:
        text = rec.get(k, "")
        if split:
            sents = [ids for ids in (_TOK.tokenize(s) for s in split_sentences(text, keep_nl)) if ids]
            if eod and sents:
                sents[-1].append(_TOK.eod)
            out[k] = sents
        else:
            ids = _TOK.tokenize(text)
            if eod and ids:
                ids.append(_TOK.eod)
            out[k] = ids
    return out, len(line)


def _lines(paths: List[str]) -> Iterator[str]:
    for p in paths:
        opener = gzip.open if p.endswith(".gz") else open
        with opener(p, "rt", encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield line


def _partition_lines(paths: List[str], part: int, parts: int, sequential: bool, total: int) -> Iterator[str]:
    if parts == 1:
        yield from _lines(paths)
        return
    per = -(-total // parts)
    for i, line in enumerate(_lines(paths)):
        if (i // per if sequential else i % parts) == part:
            yield line


def _run_partition(a, paths, part, total, prefix, level):
    from loongforge_b200.data.indexed_dataset import IndexedDatasetWriter
    dtype = np.int32 if _TOK.vocab_size > 65500 else np.uint16
    writers = {k: IndexedDatasetWriter(f"{prefix}_{k}_{level}", dtype) for k in a.json_keys}
    jobs = ((line, a.json_keys, a.append_eod, a.split_sentences, a.keep_newlines)
            for line in _partition_lines(paths, part, a.partitions, a.keep_sequential_samples, total))
    pool = None
    if a.workers > 1:
        pool = mp.Pool(a.workers, initializer=_init, initargs=(a.tokenizer_type, a.hf_tokenizer_path))
        results = pool.imap(_encode, jobs, chunksize=64)
    else:
        results = map(_encode, jobs)
    n_docs = n_tok = n_bytes = 0
    t0 = time.time()
    for enc, nb in results:
        for k, ids in enc.items():
            if not ids:
                continue
            if a.split_sentences:
                writers[k].add_sentences(ids)
                n_tok += sum(len(s) for s in ids)
            else:
                writers[k].add_document(ids)
                n_tok += len(ids)
        n_docs += 1
        n_bytes += nb
        if a.log_interval and n_docs % a.log_interval == 0:
            dt = max(time.time() - t0, 1e-9)
            print(f"partition {part}: {n_docs} documents ({n_docs / dt:.0f} docs/s, {n_bytes / dt / 2 ** 20:.2f} MB/s)", flush=True)
    if pool is not None:
        pool.close()
        pool.join()
    for w in writers.values():
        w.finalize()
    return n_docs, n_tok


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    g = p.add_argument_group("input data")
    g.add_argument("--input", required=True)
    g.add_argument("--json-keys", nargs="+", default=["text"])
    g.add_argument("--split-sentences", action="store_true")
    g.add_argument("--keep-newlines", action="store_true")
    g = p.add_argument_group("tokenizer")
    g.add_argument("--tokenizer-type", default="ByteTokenizer")
    g.add_argument("--hf-tokenizer-path", default=None)
    g.add_argument("--tokenizer-model", default=None, help="SentencePiece model (alias of --hf-tokenizer-path for that type)")
    g.add_argument("--append-eod", action="store_true")
    for flag in ("--model-family", "--vocab-file", "--merge-file", "--lang", "--additional-special-tokens"):
        g.add_argument(flag, default=None, help="accepted for launcher compatibility")
    g.add_argument("--vocab-size", type=int, default=None)
    g.add_argument("--seq-length", type=int, default=None)
    g.add_argument("--use-fast-tokenizer", action="store_true")
    g.add_argument("--split-special-tokens", action="store_true")
    g = p.add_argument_group("output / runtime")
    g.add_argument("--output-prefix", required=True)
    g.add_argument("--workers", type=int, default=1)
    g.add_argument("--partitions", type=int, default=1)
    g.add_argument("--log-interval", type=int, default=0)
    g.add_argument("--keep-sequential-samples", action="store_true")
    a = p.parse_args(argv)
    a.hf_tokenizer_path = a.hf_tokenizer_path or a.tokenizer_model
    from loongforge_b200.data.indexed_dataset import IndexedDatasetWriter

    paths = sorted(glob.glob(a.input)) or [a.input]
    _init(a.tokenizer_type, a.hf_tokenizer_path)
    os.makedirs(os.path.dirname(os.path.abspath(a.output_prefix)), exist_ok=True)
    level = "sentence" if a.split_sentences else "document"
    if a.partitions == 1:
        n_docs, n_tok = _run_partition(a, paths, 0, 0, a.output_prefix, level)
    else:
        total = sum(1 for _ in _lines(paths))
        n_docs = n_tok = 0
        for part in range(a.partitions):
            pre = f"{a.output_prefix}_part{part:03d}"
            if all(os.path.isfile(f"{pre}_{k}_{level}.idx") for k in a.json_keys):
                print(f"partition {part}: found, not redone", flush=True)
                continue
            d, t = _run_partition(a, paths, part, total, pre, level)
            n_docs, n_tok = n_docs + d, n_tok + t
        dtype = np.int32 if _TOK.vocab_size > 65500 else np.uint16
        for k in a.json_keys:
            w = IndexedDatasetWriter(f"{a.output_prefix}_{k}_{level}", dtype)
            for part in range(a.partitions):
                w.merge(f"{a.output_prefix}_part{part:03d}_{k}_{level}")
            w.finalize()
            for part in range(a.partitions):
                for ext in (".bin", ".idx"):
                    os.remove(f"{a.output_prefix}_part{part:03d}_{k}_{level}{ext}")
    print(f"processed {n_docs} documents, {n_tok} tokens -> {a.output_prefix}_*_{level}.{{bin,idx}}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
