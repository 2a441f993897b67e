"""jsonl -> Megatron ``.bin`` / ``.idx`` pre-training data (one document per line, text under
``--json-keys``, an end-of-document token appended with ``--append-eod``). Same role and flags as the
reference's tools/data_preprocess/llm/preprocess_pretrain_data.py.

    python -m tools.data_preprocess.preprocess_pretrain_data --input corpus.jsonl --output-prefix out/corpus \
        --tokenizer-type HFTokenizer --hf-tokenizer-path <dir> --append-eod [--workers 8]
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_TOK = None


def _init(tok_type, path):
    global _TOK
    from loongforge_b200.tokenizer.tokenizer import build_tokenizer
    _TOK = build_tokenizer(tok_type, path)


def _encode(args):
    line, keys, eod = args
    try:
        rec = json.loads(line)
    except json.JSONDecodeError:
        return {}
    out = {}
    for k in keys:
        ids = _TOK.tokenize(rec.get(k, ""))
        if eod and ids:
            ids.append(_TOK.eod)
        out[k] = ids
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True)
    p.add_argument("--output-prefix", required=True)
    p.add_argument("--json-keys", nargs="+", default=["text"])
    p.add_argument("--tokenizer-type", default="ByteTokenizer")
    p.add_argument("--hf-tokenizer-path", default=None)
    p.add_argument("--append-eod", action="store_true")
    p.add_argument("--workers", type=int, default=1)
    a = p.parse_args(argv)
    from loongforge_b200.data.indexed_dataset import IndexedDatasetWriter

    _init(a.tokenizer_type, a.hf_tokenizer_path)
    dtype = np.int32 if _TOK.vocab_size > 65500 else np.uint16
    os.makedirs(os.path.dirname(os.path.abspath(a.output_prefix)), exist_ok=True)
    writers = {k: IndexedDatasetWriter(f"{a.output_prefix}_{k}_document", dtype) for k in a.json_keys}
    n_docs = n_tok = 0
    with open(a.input) as f:
        jobs = ((line, a.json_keys, a.append_eod) for line in f if line.strip())
        if a.workers > 1:
            pool = mp.Pool(a.workers, initializer=_init, initargs=(a.tokenizer_type, a.hf_tokenizer_path))
            results = pool.imap(_encode, jobs, chunksize=64)
        else:
            results = map(_encode, jobs)
        for enc in results:
            for k, ids in enc.items():
                if ids:
                    writers[k].add_document(ids)
                    n_tok += len(ids)
            n_docs += 1
    for w in writers.values():
        w.finalize()
    print(f"processed {n_docs} documents, {n_tok} tokens -> {a.output_prefix}_*_document.{{bin,idx}}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
