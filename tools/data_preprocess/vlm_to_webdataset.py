"""Image-text records -> WebDataset-style tar shards (``{key}.jpg`` / ``{key}.json`` member pairs, a shard index), the
on-disk format the multimodal loaders of the reference read through Energon (reference: tools/data_preprocess VLM ->
WebDataset conversion)."""
from __future__ import annotations

import argparse
import io
import json
import os
import tarfile
from typing import Iterable


def _add(tar: tarfile.TarFile, name: str, data: bytes) -> None:
    info = tarfile.TarInfo(name)
    info.size = len(data)
    tar.addfile(info, io.BytesIO(data))


def write_shards(records: Iterable[dict], out_dir: str, image_root: str = "", samples_per_shard: int = 1000) -> dict:
    """records: ``{"image": path or [paths], "video": path or [paths], "conversations": [...]}`` (videos keep their
    container, e.g. ``.mp4``; the loader decodes frames). Returns the shard index."""
    os.makedirs(out_dir, exist_ok=True)
    index, shard, n, tar = {"shards": []}, -1, 0, None
    for i, rec in enumerate(records):
        if tar is None or n >= samples_per_shard:
            if tar is not None:
                tar.close()
                index["shards"][-1]["count"] = n
            shard, n = shard + 1, 0
            name = f"shard-{shard:06d}.tar"
            tar = tarfile.open(os.path.join(out_dir, name), "w")
            index["shards"].append({"name": name, "count": 0})
        key = f"{i:09d}"
        images = rec.get("image") or []
        images = [images] if isinstance(images, str) else list(images)
        for j, p in enumerate(images):
            with open(os.path.join(image_root, p), "rb") as f:
                ext = os.path.splitext(p)[1].lstrip(".").lower() or "jpg"
                _add(tar, f"{key}.{j}.{ext}" if len(images) > 1 else f"{key}.{ext}", f.read())
        videos = rec.get("video") or rec.get("videos") or []
        videos = [videos] if isinstance(videos, str) else list(videos)
        for j, p in enumerate(videos):
            with open(os.path.join(image_root, p), "rb") as f:
                ext = os.path.splitext(p)[1].lstrip(".").lower() or "mp4"
                _add(tar, f"{key}.v{j}.{ext}", f.read())
        meta = {k: v for k, v in rec.items() if k not in ("image", "video", "videos")}
        meta["num_images"], meta["num_videos"] = len(images), len(videos)
        _add(tar, f"{key}.json", json.dumps(meta).encode())
        n += 1
    if tar is not None:
        tar.close()
        index["shards"][-1]["count"] = n
    index["total"] = sum(s["count"] for s in index["shards"])
    with open(os.path.join(out_dir, "index.json"), "w") as f:
        json.dump(index, f)
    return index


def read_shard(path: str):
    """Yields ``(key, {extension: bytes})`` groups in order — the reader side used by tests and simple loaders."""
    cur, group = None, {}
    with tarfile.open(path) as tar:
        for m in tar:
            key, _, ext = m.name.partition(".")
            if key != cur and cur is not None:
                yield cur, group
                group = {}
            cur = key
            group[ext] = tar.extractfile(m).read()
    if cur is not None:
        yield cur, group


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True, help="JSON / JSONL with image + conversations records")
    ap.add_argument("--image-root", default="")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--samples-per-shard", type=int, default=1000)
    args = ap.parse_args(argv)
    from tools.data_preprocess.preprocess_sft_data import iter_records
    return write_shards(iter_records(args.input), args.output_dir, args.image_root, args.samples_per_shard)


if __name__ == "__main__":
    main()
