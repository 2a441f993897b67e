"""Offline packing of image-text shards in three resumable stages (the role of the reference's
tools/data_preprocess/vlm/offline_packing pipeline: scan manifest -> build plan -> write shards):

    python -m tools.data_preprocess.vlm_offline_packing scan  --shards SRC_DIR --manifest m.sqlite [--patch 14 --merge 2]
    python -m tools.data_preprocess.vlm_offline_packing plan  --manifest m.sqlite --seq-length 4096 [--bucket-width 64]
    python -m tools.data_preprocess.vlm_offline_packing write --shards SRC_DIR --manifest m.sqlite --output-dir DST_DIR
    python -m tools.data_preprocess.vlm_offline_packing all   --shards SRC_DIR --output-dir DST_DIR --seq-length 4096

* scan: one pass over the source shards (the layout of ``vlm_to_webdataset.py``); per sample the text length (a
  tokenizer when ``--tokenizer`` is given, else a whitespace / punctuation estimate) and the number of image tokens after
  the vision tower's resize and spatial merge go into an SQLite manifest. Only image HEADERS are read.
* plan: hash-bucket packing (``offline_packing.pack_with_buckets``) over the manifest's lengths; the pack id of every
  sample and the fill rate are stored in the manifest. Samples longer than the sequence length are marked dropped.
* write: samples are copied pack by pack into new shards, every member's JSON gets ``pack_id`` / ``pack_size``, and the
  shard index carries ``"packed": true`` with the sequence length: a loader that sees it keeps each pack together
  (``loongforge_b200.data.multimodal.webdataset_samples(..., keep_packs=True)``) instead of packing online.
"""
from __future__ import annotations

import argparse
import io
import json
import os
import re
import sqlite3
import sys
import tarfile
from typing import Dict, Iterator, List, Optional, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _image_size(data: bytes, ext: str) -> Tuple[int, int]:
    """(height, width) from the file header (``.npy``: from the array header)."""
    if ext.endswith("npy"):
        import numpy as np
        arr = np.load(io.BytesIO(data), mmap_mode=None, allow_pickle=False)
        return int(arr.shape[0]), int(arr.shape[1])
    from PIL import Image
    with Image.open(io.BytesIO(data)) as im:
        w, h = im.size
    return h, w


def _text_length(meta: dict, tokenize=None) -> int:
    conv = meta.get("conversation") or meta.get("conversations") or []
    text = " ".join(str(c.get("content", c.get("value", ""))) for c in conv).replace("<image>", " ")
    if tokenize is not None:
        return len(tokenize(text)) + 2 * len(conv)
    # without a tokenizer: words and punctuation marks, a slight over-estimate for sub-word vocabularies
    return int(1.3 * len(re.findall(r"\w+|[^\w\s]", text))) + 4 * len(conv)


def iter_source(shards_dir: str) -> Iterator[Tuple[str, str, Dict[str, bytes]]]:
    from tools.data_preprocess.vlm_to_webdataset import read_shard
    with open(os.path.join(shards_dir, "index.json")) as f:
        names = [s["name"] for s in json.load(f)["shards"]]
    for name in names:
        for key, group in read_shard(os.path.join(shards_dir, name)):
            yield name, key, group


def _db(path: str) -> sqlite3.Connection:
    con = sqlite3.connect(path)
    con.execute("CREATE TABLE IF NOT EXISTS samples (key TEXT PRIMARY KEY, shard TEXT, text_len INTEGER, "
                "image_tokens INTEGER, total_len INTEGER, pack_id INTEGER)")
    con.execute("CREATE TABLE IF NOT EXISTS meta (k TEXT PRIMARY KEY, v TEXT)")
    return con


def scan(shards_dir: str, manifest: str, patch: int = 14, merge: int = 2, min_pixels: Optional[int] = None,
         max_pixels: Optional[int] = None, tokenize=None) -> int:
    from loongforge_b200.data.multimodal import VisionPreprocess
    kw = {k: v for k, v in (("min_pixels", min_pixels), ("max_pixels", max_pixels)) if v}
    vis = VisionPreprocess(patch_size=patch, merge_size=merge, **kw)
    con = _db(manifest)
    done = {r[0] for r in con.execute("SELECT key FROM samples")}  # resumable: scanned samples are skipped
    n = 0
    for shard, key, group in iter_source(shards_dir):
        if key in done:
            continue
        meta = json.loads(group["json"])
        img_tokens = 0
        for ext, data in group.items():
            if ext == "json":
                continue
            h, w = _image_size(data, ext)
            hb, wb = vis.smart_resize(h, w)
            img_tokens += (hb // patch // merge) * (wb // patch // merge)
        tl = _text_length(meta, tokenize)
        con.execute("INSERT OR REPLACE INTO samples VALUES (?, ?, ?, ?, ?, NULL)", (key, shard, tl, img_tokens, tl + img_tokens))
        n += 1
        if n % 1000 == 0:
            con.commit()
    con.commit()
    con.close()
    return n


def plan(manifest: str, seq_length: int, bucket_width: int = 64) -> dict:
    from tools.data_preprocess.offline_packing import pack_with_buckets
    con = _db(manifest)
    rows = con.execute("SELECT key, total_len FROM samples ORDER BY key").fetchall()
    keys, lengths = [r[0] for r in rows], [int(r[1]) for r in rows]
    packs = pack_with_buckets(lengths, seq_length, bucket_width)
    con.execute("UPDATE samples SET pack_id = NULL")
    for pid, p in enumerate(packs):
        con.executemany("UPDATE samples SET pack_id = ? WHERE key = ?", [(pid, keys[i]) for i in p])
    used = sum(lengths[i] for p in packs for i in p)
    stats = {"seq_length": seq_length, "packs": len(packs), "samples": len(keys),
             "dropped": len(keys) - sum(len(p) for p in packs),
             "fill_rate": used / max(len(packs) * seq_length, 1)}
    con.execute("INSERT OR REPLACE INTO meta VALUES ('plan', ?)", (json.dumps(stats),))
    con.commit()
    con.close()
    return stats


def write(shards_dir: str, manifest: str, output_dir: str, packs_per_shard: int = 256) -> dict:
    con = _db(manifest)
    stats = json.loads(con.execute("SELECT v FROM meta WHERE k = 'plan'").fetchone()[0])
    pack_of = {k: p for k, p in con.execute("SELECT key, pack_id FROM samples WHERE pack_id IS NOT NULL")}
    size_of: Dict[int, int] = {}
    for p in pack_of.values():
        size_of[p] = size_of.get(p, 0) + 1
    con.close()
    # one pass over the source collects every planned sample's members; packs are then written in pack order
    by_pack: Dict[int, List[Tuple[str, Dict[str, bytes]]]] = {}
    for _, key, group in iter_source(shards_dir):
        if key in pack_of:
            by_pack.setdefault(pack_of[key], []).append((key, group))
    os.makedirs(output_dir, exist_ok=True)
    index = {"shards": [], "packed": True, "seq_length": stats["seq_length"], "fill_rate": stats["fill_rate"]}
    tar, in_shard, count = None, 0, 0
    for pid in sorted(by_pack):
        if tar is None or in_shard >= packs_per_shard:
            if tar is not None:
                tar.close()
                index["shards"][-1]["count"] = count
            name = f"packed-{len(index['shards']):06d}.tar"
            tar = tarfile.open(os.path.join(output_dir, name), "w")
            index["shards"].append({"name": name, "count": 0})
            in_shard, count = 0, 0
        for key, group in sorted(by_pack[pid]):
            meta = json.loads(group["json"])
            meta.update(pack_id=pid, pack_size=size_of[pid])
            for ext, data in group.items():
                payload = json.dumps(meta).encode() if ext == "json" else data
                info = tarfile.TarInfo(f"{key}.{ext}")
                info.size = len(payload)
                tar.addfile(info, io.BytesIO(payload))
            count += 1
        in_shard += 1
    if tar is not None:
        tar.close()
        index["shards"][-1]["count"] = count
    index["total"] = sum(s["count"] for s in index["shards"])
    index["packs"] = len(by_pack)
    with open(os.path.join(output_dir, "index.json"), "w") as f:
        json.dump(index, f)
    return index


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("stage", choices=["scan", "plan", "write", "all"])
    ap.add_argument("--shards", default=None)
    ap.add_argument("--manifest", default=None)
    ap.add_argument("--output-dir", default=None)
    ap.add_argument("--seq-length", type=int, default=4096)
    ap.add_argument("--bucket-width", type=int, default=64)
    ap.add_argument("--patch", type=int, default=14)
    ap.add_argument("--merge", type=int, default=2)
    ap.add_argument("--min-pixels", type=int, default=None)
    ap.add_argument("--max-pixels", type=int, default=None)
    ap.add_argument("--packs-per-shard", type=int, default=256)
    ap.add_argument("--tokenizer", default=None, help="Hugging Face tokenizer directory for exact text lengths")
    a = ap.parse_args(argv)
    manifest = a.manifest or (os.path.join(a.output_dir, "manifest.sqlite") if a.output_dir else None)
    if manifest is None:
        ap.error("--manifest (or --output-dir) is needed")
    if a.output_dir:
        os.makedirs(a.output_dir, exist_ok=True)
    tokenize = None
    if a.tokenizer:
        from loongforge_b200.tokenizer.tokenizer import build_tokenizer
        tokenize = build_tokenizer("HFTokenizer", a.tokenizer).tokenize
    out = {}
    if a.stage in ("scan", "all"):
        out["scanned"] = scan(a.shards, manifest, a.patch, a.merge, a.min_pixels, a.max_pixels, tokenize)
    if a.stage in ("plan", "all"):
        out["plan"] = plan(manifest, a.seq_length, a.bucket_width)
    if a.stage in ("write", "all"):
        out["index"] = write(a.shards, manifest, a.output_dir, a.packs_per_shard)
    print(json.dumps({k: (v if not isinstance(v, dict) else {kk: vv for kk, vv in v.items() if kk != "shards"})
                      for k, v in out.items()}))
    return out


if __name__ == "__main__":
    main()
