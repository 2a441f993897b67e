"""Offline sequence packing with hash buckets: samples are bucketed by length so that packing a corpus that does not fit
in memory needs only the length index; each bucket is filled first-fit from the longest bucket down (reference:
tools/data_preprocess offline packing, hash-bucket variant).

Input: the ``index.json`` written by ``preprocess_sft_data.py`` (``--split`` picks the split) or any JSON with a ``lengths`` list.
Output: ``packs.json`` — a list of packs, each a list of sample ids whose lengths sum to at most ``--seq-length``."""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from typing import Dict, List


def pack_with_buckets(lengths: List[int], capacity: int, bucket_width: int = 64) -> List[List[int]]:
    buckets: Dict[int, List[int]] = defaultdict(list)
    for i, n in enumerate(lengths):
        if n <= capacity:
            buckets[n // bucket_width].append(i)
    keys = sorted(buckets, reverse=True)
    packs: List[List[int]] = []
    while True:
        # open a pack with the longest remaining sample
        first = next((k for k in keys if buckets[k]), None)
        if first is None:
            break
        i = buckets[first].pop()
        pack, room = [i], capacity - lengths[i]
        # then repeatedly take a sample from the fullest-fitting bucket
        while room > 0:
            k = next((k for k in keys if buckets[k] and k * bucket_width <= room), None)
            if k is None:
                break
            # within the bucket lengths vary by < bucket_width: check the actual fit
            j = next((idx for idx in range(len(buckets[k]) - 1, -1, -1) if lengths[buckets[k][idx]] <= room), None)
            if j is None:
                # nothing in this bucket fits exactly; try lower buckets
                lower = next((kk for kk in keys if kk < k and buckets[kk]), None)
                if lower is None:
                    break
                k, j = lower, len(buckets[lower]) - 1
                if lengths[buckets[k][j]] > room:
                    break
            s = buckets[k].pop(j)
            pack.append(s)
            room -= lengths[s]
        packs.append(pack)
    return packs


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--index", required=True)
    ap.add_argument("--seq-length", type=int, required=True)
    ap.add_argument("--bucket-width", type=int, default=64)
    ap.add_argument("--output", required=True)
    ap.add_argument("--split", default="train", help="split of an index written by preprocess_sft_data.py")
    args = ap.parse_args(argv)
    with open(args.index) as f:
        node = json.load(f)
    lengths = node["lengths"] if "lengths" in node else node["splits"][args.split]["lengths"]
    packs = pack_with_buckets(lengths, args.seq_length, args.bucket_width)
    used = sum(lengths[i] for p in packs for i in p)
    with open(args.output, "w") as f:
        json.dump({"seq_length": args.seq_length, "packs": packs,
                   "fill_rate": used / max(len(packs) * args.seq_length, 1)}, f)
    return packs


if __name__ == "__main__":
    main()
