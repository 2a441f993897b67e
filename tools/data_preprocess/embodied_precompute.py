"""Pre-computes what the frozen parts of a world-model policy produce, once per data set, so that training does not run
the video codec, the text encoder and the image tower on every step.

    python -m tools.data_preprocess.embodied_precompute build    --output CACHE [--config recipe.yaml] key=value ...
    python -m tools.data_preprocess.embodied_precompute validate --cache CACHE [--deep]

``build`` walks the data set of the recipe in index order and stores, per sample, the video latents of the policy's codec,
the instruction embedding (+ mask) of its text encoder and, for DreamZero, the image tokens of the observed frame, in
shards ``features_00000.npz`` (arrays stacked over the shard's samples) next to ``manifest.json``: sample count, shard
table, array shapes and dtypes, and a fingerprint of the frozen weights and of the data-set arguments. An interrupted build
resumes after the last complete shard. ``validate`` checks the manifest against the shards (presence, counts, shapes,
finite values with ``--deep``) and — given the recipe arguments — that the fingerprint still matches.

Training reads the cache with ``precomputed_cache: CACHE`` (``loongforge_b200.embodied.data.PrecomputedFeatures``): samples
gain ``latents`` / ``text_emb`` / ``text_emb_mask`` / ``image_tokens`` and lose the raw video.

(reference: tools/data_preprocess/embodied/dreamzero/precompute_features.py, cache_precompute/{features,storage}.py,
validate_precomputed_feature_artifact.py; loongforge/embodied/data/datasets/lingbot_va/latent_lerobot_dataset.py)
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Dict, List

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MANIFEST = "manifest.json"


def frozen_modules(policy) -> Dict[str, torch.nn.Module]:
    inner = getattr(policy, "policy", policy)
    return {n: getattr(inner, n) for n in ("vae", "text_encoder", "image_tower") if hasattr(inner, n)}


def fingerprint(policy, args) -> str:
    """Hash of the frozen modules' weights and of the arguments that decide what a sample is."""
    h = hashlib.sha256()
    for name, mod in sorted(frozen_modules(policy).items()):
        for k, v in sorted(mod.state_dict().items()):
            h.update(f"{name}.{k}".encode())
            h.update(v.detach().cpu().float().numpy().tobytes())
    for k in ("dataset_type", "dataset_path", "video_frames", "video_frame_stride", "image_size", "max_text_len", "model_name"):
        h.update(f"{k}={getattr(args, k, None)}".encode())
    return h.hexdigest()[:32]


@torch.no_grad()
def features_of(policy, batch: Dict[str, torch.Tensor], dtype=np.float16) -> Dict[str, np.ndarray]:
    from loongforge_b200.embodied.wan_blocks import video_from_batch
    inner = getattr(policy, "policy", policy)
    out: Dict[str, np.ndarray] = {}
    frames = inner.c.video_frames
    video = video_from_batch(batch, frames)
    if hasattr(inner, "vae"):
        out["latents"] = inner.vae.encode(video).float().cpu().numpy().astype(dtype)
    if hasattr(inner, "text_encoder"):
        tok = batch["tokens"] if "tokens" in batch else batch["text"]
        mask = tok != 0
        keep = mask.clone()
        keep[:, 0] = True
        out["text_emb"] = inner.text_encoder(tok, mask).float().cpu().numpy().astype(dtype)
        out["text_emb_mask"] = keep.cpu().numpy()
    if hasattr(inner, "image_tower"):
        out["image_tokens"] = inner.image_tower(video[:, :, 0]).float().cpu().numpy().astype(dtype)
    return out


def build(args, output: str, shard_size: int = 256, batch_size: int = 8, dtype: str = "float16", policy=None, dataset=None) -> dict:
    from loongforge_b200.embodied.data import _base_dataset, collate
    from loongforge_b200.embodied.models import build_policy
    torch.manual_seed(args.seed)
    policy = (policy or build_policy(args.model_name, args)).eval()
    ds = dataset or _base_dataset(args)
    os.makedirs(output, exist_ok=True)
    fp = fingerprint(policy, args)
    path = os.path.join(output, MANIFEST)
    manifest = {"fingerprint": fp, "model_name": args.model_name, "num_samples": len(ds), "shard_size": shard_size, "dtype": dtype,
                "shards": [], "arrays": {}, "complete": False}
    if os.path.isfile(path):
        old = json.load(open(path))
        if old.get("fingerprint") == fp and old.get("shard_size") == shard_size and old.get("num_samples") == len(ds):
            manifest = old   # resume: the shards listed there are complete
    done = len(manifest["shards"])
    np_dtype = np.dtype(dtype)
    for s in range(done, -(-len(ds) // shard_size)):
        lo, hi = s * shard_size, min((s + 1) * shard_size, len(ds))
        parts: Dict[str, List[np.ndarray]] = {}
        for b in range(lo, hi, batch_size):
            batch = collate([ds[i] for i in range(b, min(b + batch_size, hi))])
            for k, v in features_of(policy, batch, np_dtype).items():
                parts.setdefault(k, []).append(v)
        arrays = {k: np.concatenate(v) for k, v in parts.items()}
        name = f"features_{s:05d}.npz"
        tmp = os.path.join(output, name + ".tmp.npz")
        np.savez(tmp, **arrays)
        os.replace(tmp, os.path.join(output, name))
        manifest["shards"].append({"file": name, "first": lo, "count": hi - lo})
        manifest["arrays"] = {k: {"shape": list(v.shape[1:]), "dtype": str(v.dtype)} for k, v in arrays.items()}
        with open(path + ".tmp", "w") as f:
            json.dump(manifest, f)
        os.replace(path + ".tmp", path)
    manifest["complete"] = True
    with open(path, "w") as f:
        json.dump(manifest, f, indent=1)
    return manifest


def validate(cache: str, deep: bool = False, expected_fingerprint: str = None) -> List[str]:
    """Problems found (empty list: the cache is usable)."""
    problems: List[str] = []
    path = os.path.join(cache, MANIFEST)
    if not os.path.isfile(path):
        return [f"{path} is missing"]
    m = json.load(open(path))
    if not m.get("complete"):
        problems.append("the build did not finish (complete = false)")
    if expected_fingerprint and m.get("fingerprint") != expected_fingerprint:
        problems.append(f"fingerprint {m.get('fingerprint')} != expected {expected_fingerprint}: frozen weights or data arguments changed")
    nxt = 0
    for sh in m.get("shards", []):
        f = os.path.join(cache, sh["file"])
        if sh["first"] != nxt:
            problems.append(f"{sh['file']}: starts at sample {sh['first']}, expected {nxt}")
        nxt = sh["first"] + sh["count"]
        if not os.path.isfile(f):
            problems.append(f"{sh['file']} is missing")
            continue
        with np.load(f) as z:
            for k, spec in m["arrays"].items():
                if k not in z.files:
                    problems.append(f"{sh['file']}: array {k} is missing")
                    continue
                a = z[k]
                if list(a.shape[1:]) != spec["shape"] or a.shape[0] != sh["count"] or str(a.dtype) != spec["dtype"]:
                    problems.append(f"{sh['file']}: {k} has shape {a.shape} / {a.dtype}, manifest says [{sh['count']}, *{spec['shape']}] / {spec['dtype']}")
                elif deep and a.dtype.kind == "f" and not np.isfinite(a.astype(np.float32)).all():
                    problems.append(f"{sh['file']}: {k} holds non-finite values")
    if nxt != m.get("num_samples"):
        problems.append(f"shards cover {nxt} samples of {m.get('num_samples')}")
    return problems


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build")
    b.add_argument("--output", required=True)
    b.add_argument("--config", default=None)
    b.add_argument("--shard-size", type=int, default=256)
    b.add_argument("--batch-size", type=int, default=8)
    b.add_argument("--dtype", default="float16", choices=["float16", "float32"])
    b.add_argument("overrides", nargs="*")
    v = sub.add_parser("validate")
    v.add_argument("--cache", required=True)
    v.add_argument("--deep", action="store_true")
    v.add_argument("--config", default=None)
    v.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    from loongforge_b200.embodied.config import parse_args
    if a.cmd == "build":
        args = parse_args((["--config", a.config] if a.config else []) + list(a.overrides))
        m = build(args, a.output, a.shard_size, a.batch_size, a.dtype)
        print(json.dumps({"samples": m["num_samples"], "shards": len(m["shards"]), "arrays": m["arrays"], "fingerprint": m["fingerprint"]}))
        return 0
    expected = None
    if a.config or a.overrides:
        from loongforge_b200.embodied.models import build_policy
        args = parse_args((["--config", a.config] if a.config else []) + list(a.overrides))
        torch.manual_seed(args.seed)
        expected = fingerprint(build_policy(args.model_name, args), args)
    problems = validate(a.cache, a.deep, expected)
    print(json.dumps({"ok": not problems, "problems": problems}))
    return 0 if not problems else 1


if __name__ == "__main__":
    sys.exit(main())
