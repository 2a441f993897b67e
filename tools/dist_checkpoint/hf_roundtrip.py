"""Round-trip check of the Hugging Face bridge (the role of the reference's
tools/dist_checkpoint/checkpoint/hf_roundtrip_test.py): Hugging Face weights -> torch_dist checkpoint -> Hugging Face
weights, then every tensor of the result is compared with the source.

    python -m tools.dist_checkpoint.hf_roundtrip --hf-dir HF_DIR --family llama3 --model-name llama3-8b \\
        [--work-dir DIR] [--atol 0] [--keep] [--report report.json]
    python -m tools.dist_checkpoint.hf_roundtrip --synthetic --family qwen3_moe --model-name tiny-qwen3-moe
        (no source checkpoint at hand: random weights of the preset are exported first and used as the source)

Exit code 0 when every tensor matches (bit-exact by default), 1 otherwise. The report lists missing / extra names, shape
mismatches and the largest absolute difference per tensor that differs.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
import tempfile
from typing import Dict

import torch


def compare_state_dicts(a: Dict[str, torch.Tensor], b: Dict[str, torch.Tensor], atol: float = 0.0) -> dict:
    rep = {"missing_in_result": sorted(set(a) - set(b)), "extra_in_result": sorted(set(b) - set(a)),
           "shape_mismatch": [], "value_mismatch": [], "compared": 0}
    for k in sorted(set(a) & set(b)):
        x, y = a[k], b[k]
        if tuple(x.shape) != tuple(y.shape):
            rep["shape_mismatch"].append({"name": k, "source": list(x.shape), "result": list(y.shape)})
            continue
        rep["compared"] += 1
        if x.dtype != y.dtype or not torch.equal(x, y):
            d = (x.float() - y.float()).abs().max().item() if x.numel() else 0.0
            if d > atol or x.dtype != y.dtype:
                rep["value_mismatch"].append({"name": k, "max_abs_diff": d, "source_dtype": str(x.dtype),
                                              "result_dtype": str(y.dtype)})
    rep["ok"] = not (rep["missing_in_result"] or rep["extra_in_result"] or rep["shape_mismatch"] or rep["value_mismatch"])
    return rep


def synthetic_source(hf_dir: str, family: str, model_name: str, seed: int = 0) -> None:
    """Random weights of the preset, written in Hugging Face layout (through the same name map, from the framework's
    side), so that the round trip can run without a downloaded checkpoint."""
    from loongforge_b200.ckpt.hf_bridge import hf_config_from_model
    from loongforge_b200.models.gpt import GPTModel
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from tools.convert_checkpoint import name_maps as nm
    from tools.convert_checkpoint.convert import save_hf
    from tools.dist_checkpoint.convert_dist_checkpoint import _dims

    cfg = get_model_config(model_name)
    cfg.pad_vocab(1)
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(ps.ParallelDims())
    torch.manual_seed(seed)
    model = GPTModel(cfg)
    mc = {k: v.detach().clone() for k, v in model.state_dict().items() if torch.is_tensor(v) and "_extra_state" not in k}
    margs = {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in vars(cfg).items()}
    hf = nm.mcore_to_hf(mc, nm.FAMILIES[family], vocab_size=cfg.vocab_size, **_dims(margs))
    save_hf(hf, hf_dir, hf_config_from_model(cfg, family))


def roundtrip(hf_dir: str, family: str, model_name: str, work_dir: str, atol: float = 0.0) -> dict:
    from tools.convert_checkpoint.convert import load_hf
    from tools.dist_checkpoint.convert_dist_checkpoint import dist_to_hf, hf_to_dist

    ckpt, back = os.path.join(work_dir, "torch_dist"), os.path.join(work_dir, "hf_back")
    n_in = hf_to_dist(hf_dir, ckpt, family, model_name)
    n_out = dist_to_hf(ckpt, back, family)
    rep = compare_state_dicts(load_hf(hf_dir), load_hf(back), atol)
    rep.update(tensors_in_checkpoint=n_in, tensors_exported=n_out, family=family, model_name=model_name)
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hf-dir", default=None)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--family", required=True)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--work-dir", default=None)
    ap.add_argument("--atol", type=float, default=0.0)
    ap.add_argument("--keep", action="store_true", help="keep the intermediate checkpoint and the re-exported weights")
    ap.add_argument("--report", default=None)
    a = ap.parse_args(argv)
    if not a.synthetic and not a.hf_dir:
        ap.error("give --hf-dir or --synthetic")
    work = a.work_dir or tempfile.mkdtemp(prefix="hf_roundtrip_")
    os.makedirs(work, exist_ok=True)
    try:
        src = a.hf_dir
        if a.synthetic:
            src = os.path.join(work, "hf_source")
            synthetic_source(src, a.family, a.model_name)
        rep = roundtrip(src, a.family, a.model_name, work, a.atol)
    finally:
        if not a.keep and a.work_dir is None:
            shutil.rmtree(work, ignore_errors=True)
    if a.report:
        with open(a.report, "w") as f:
            json.dump(rep, f, indent=1)
    print(json.dumps({k: (v if not isinstance(v, list) else len(v)) for k, v in rep.items()}))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
