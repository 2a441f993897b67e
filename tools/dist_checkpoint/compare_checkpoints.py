"""Tensor-by-tensor comparison of two checkpoints, each a Hugging Face directory (safetensors / .bin shards) or a
training checkpoint directory (torch_dist layout, newest iteration unless ``--iteration``):

    python -m tools.dist_checkpoint.compare_checkpoints A B [--atol 0 --rtol 0] [--report report.json] [--ignore REGEX ...]

Reports tensors only in A / only in B, shape or dtype differences, and for the common ones the largest absolute and
relative difference and the cosine similarity; exit code 1 when anything differs beyond the tolerances (reference:
tools/dist_checkpoint/utils/comparison_utils.py:18-307).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
import sys
from typing import Dict, List, Optional

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_any(path: str, iteration: Optional[int] = None) -> Dict[str, torch.Tensor]:
    if os.path.isfile(path):
        if path.endswith(".safetensors"):
            from safetensors.torch import load_file
            return load_file(path)
        blob = torch.load(path, map_location="cpu", weights_only=False)
        return blob.get("model", blob) if isinstance(blob, dict) else blob
    st = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if st:
        from safetensors.torch import load_file
        out: Dict[str, torch.Tensor] = {}
        for f in st:
            out.update(load_file(f))
        return out
    bins = sorted(glob.glob(os.path.join(path, "pytorch_model*.bin")))
    if bins:
        out = {}
        for f in bins:
            out.update(torch.load(f, map_location="cpu", weights_only=False))
        return out
    from tools.dist_checkpoint.convert_dist_checkpoint import read_model_tensors
    return read_model_tensors(path, iteration)[0]


def compare(a: Dict[str, torch.Tensor], b: Dict[str, torch.Tensor], atol: float = 0.0, rtol: float = 0.0,
            ignore: Optional[List[str]] = None) -> dict:
    pats = [re.compile(p) for p in (ignore or [])]
    skip = lambda k: any(p.search(k) for p in pats)  # noqa: E731
    ka, kb = {k for k in a if not skip(k)}, {k for k in b if not skip(k)}
    rep = {"only_in_a": sorted(ka - kb), "only_in_b": sorted(kb - ka), "shape_mismatch": [], "dtype_mismatch": [],
           "value_mismatch": [], "matched": 0, "max_abs_diff": 0.0, "worst_key": None}
    for k in sorted(ka & kb):
        x, y = a[k], b[k]
        if tuple(x.shape) != tuple(y.shape):
            rep["shape_mismatch"].append({"key": k, "a": list(x.shape), "b": list(y.shape)})
            continue
        if x.dtype != y.dtype:
            rep["dtype_mismatch"].append({"key": k, "a": str(x.dtype), "b": str(y.dtype)})
        xf, yf = x.float(), y.float()
        d = (xf - yf).abs()
        mx = float(d.max()) if d.numel() else 0.0
        if mx > rep["max_abs_diff"]:
            rep["max_abs_diff"], rep["worst_key"] = mx, k
        if not torch.allclose(xf, yf, atol=atol, rtol=rtol, equal_nan=True):
            denom = float(yf.abs().max()) or 1.0
            cos = float(torch.nn.functional.cosine_similarity(xf.flatten(), yf.flatten(), dim=0)) if xf.numel() else 1.0
            rep["value_mismatch"].append({"key": k, "max_abs": mx, "max_rel": mx / denom, "cosine": cos,
                                          "fraction_differing": float((d > atol + rtol * yf.abs()).float().mean())})
        else:
            rep["matched"] += 1
    rep["equal"] = not (rep["only_in_a"] or rep["only_in_b"] or rep["shape_mismatch"] or rep["value_mismatch"])
    return rep


def summary(rep: dict, limit: int = 10) -> str:
    L = [f"matched {rep['matched']} tensors; largest difference {rep['max_abs_diff']:.3e}" + (f" at {rep['worst_key']}" if rep["worst_key"] else "")]
    for title, key in (("only in A", "only_in_a"), ("only in B", "only_in_b")):
        if rep[key]:
            L.append(f"{title}: {len(rep[key])} (" + ", ".join(rep[key][:limit]) + (" ..." if len(rep[key]) > limit else "") + ")")
    for m in rep["shape_mismatch"][:limit]:
        L.append(f"shape  {m['key']}: {m['a']} vs {m['b']}")
    for m in rep["dtype_mismatch"][:limit]:
        L.append(f"dtype  {m['key']}: {m['a']} vs {m['b']}")
    for m in sorted(rep["value_mismatch"], key=lambda m: -m["max_abs"])[:limit]:
        L.append(f"value  {m['key']}: max abs {m['max_abs']:.3e}, max rel {m['max_rel']:.3e}, cosine {m['cosine']:.6f}, "
                 f"{100 * m['fraction_differing']:.2f}% of entries")
    L.append("EQUAL" if rep["equal"] else "DIFFERENT")
    return "\n".join(L)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("a")
    ap.add_argument("b")
    ap.add_argument("--atol", type=float, default=0.0)
    ap.add_argument("--rtol", type=float, default=0.0)
    ap.add_argument("--iteration", type=int, default=None)
    ap.add_argument("--ignore", nargs="*", default=[], help="regular expressions of tensor names to leave out")
    ap.add_argument("--report", default=None)
    x = ap.parse_args(argv)
    rep = compare(load_any(x.a, x.iteration), load_any(x.b, x.iteration), x.atol, x.rtol, x.ignore)
    print(summary(rep))
    if x.report:
        with open(x.report, "w") as f:
            json.dump(rep, f, indent=1)
    return 0 if rep["equal"] else 1


if __name__ == "__main__":
    sys.exit(main())
