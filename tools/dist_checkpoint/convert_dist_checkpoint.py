"""Offline conversion between this framework's ``torch_dist`` checkpoints and Hugging Face weights, without starting
a trainer (the role of the reference's tools/dist_checkpoint: hf_checkpoint_loader.py / hf_checkpoint_saver.py used
offline, and its roundtrip test).

A ``torch_dist`` checkpoint stores every model tensor under its layout-independent name (global layer and expert
numbers) with its unsharded shape, so the whole model can be read into plain tensors whatever parallel layout wrote it,
and a checkpoint written here from Hugging Face weights loads under any layout.

    python -m tools.dist_checkpoint.convert_dist_checkpoint --to hf   --load ckpt_dir --save hf_dir  --family llama3
    python -m tools.dist_checkpoint.convert_dist_checkpoint --to dist --load hf_dir   --save ckpt_dir --family llama3 \\
        --model-name llama3-8b
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, Optional, Tuple

import torch


def read_model_tensors(ckpt_root: str, iteration: Optional[int] = None) -> Tuple[Dict[str, torch.Tensor], dict]:
    """(unsharded model tensors, common state) of a torch_dist checkpoint directory (the one holding the tracker)."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    from loongforge_b200.ckpt.checkpointing import iteration_dir, read_tracker

    it, release = (iteration, False) if iteration is not None else read_tracker(ckpt_root)
    if it is None:
        raise FileNotFoundError(f"no checkpoint tracker under {ckpt_root}")
    d = iteration_dir(ckpt_root, it, release)
    md = FileSystemReader(d).read_metadata()
    state = {}
    for key, meta in md.state_dict_metadata.items():
        if key.startswith(("optimizer.", "rng_state")) or not isinstance(meta, TensorStorageMetadata):
            continue
        state[key] = torch.empty(tuple(meta.size), dtype=meta.properties.dtype)
    dcp.load(state, checkpoint_id=d, no_dist=True)
    common = torch.load(os.path.join(d, "common.pt"), weights_only=False)
    return state, common


def write_model_tensors(ckpt_root: str, tensors: Dict[str, torch.Tensor], model_args: dict, iteration: int = 0) -> str:
    """A weights-only torch_dist checkpoint that the trainer loads under any parallel layout (``--load`` with
    ``--finetune`` or ``--no-load-optim --no-load-rng``, or ``--pretrained-checkpoint``)."""
    import torch.distributed.checkpoint as dcp

    from loongforge_b200.ckpt.checkpointing import CHECKPOINT_VERSION, iteration_dir, write_tracker

    d = iteration_dir(ckpt_root, iteration)
    os.makedirs(d, exist_ok=True)
    dcp.save({k: v.contiguous() for k, v in tensors.items()}, checkpoint_id=d, no_dist=True)
    common = {"args": {"model": model_args, "train": {},
                       "parallel": {"tp": 1, "pp": 1, "cp": 1, "ep": 1, "dp": 1, "world": 1}},
              "checkpoint_version": CHECKPOINT_VERSION, "iteration": iteration, "consumed_samples": 0,
              "num_floating_point_operations_so_far": 0.0, "opt_param_scheduler": {}, "optimizer": {}}
    torch.save(common, os.path.join(d, "common.pt"))
    with open(os.path.join(d, "metadata.json"), "w") as f:
        json.dump({"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch"}, f)
    write_tracker(ckpt_root, iteration)
    return d


def _dims(model_args: dict) -> dict:
    g = model_args.get
    return dict(num_layers=g("num_layers"), num_heads=g("num_attention_heads"),
                num_groups=g("num_query_groups") or g("num_attention_heads"), num_experts=g("num_moe_experts"),
                tie_embeddings=not g("untie_embeddings_and_output_weights", True))


def dist_to_hf(ckpt_root: str, hf_dir: str, family: str, iteration: Optional[int] = None) -> int:
    from loongforge_b200.ckpt.hf_bridge import hf_config_from_model
    from loongforge_b200.models.config import TransformerConfig
    from tools.convert_checkpoint import name_maps as nm
    from tools.convert_checkpoint.convert import save_hf

    mc, common = read_model_tensors(ckpt_root, iteration)
    margs = common["args"]["model"]
    hf = nm.mcore_to_hf(mc, nm.FAMILIES[family], vocab_size=margs.get("vocab_size"), **_dims(margs))
    known = {f.name for f in __import__("dataclasses").fields(TransformerConfig)}
    cfg = TransformerConfig(**{k: v for k, v in margs.items() if k in known and k != "params_dtype"})
    save_hf(hf, hf_dir, hf_config_from_model(cfg, family))
    return len(hf)


def hf_to_dist(hf_dir: str, ckpt_root: str, family: str, model_name: Optional[str] = None,
               overrides: Optional[dict] = None) -> int:
    """``model_name``: a preset / YAML name of this framework that describes the architecture (sizes are checked against
    the Hugging Face tensors by the name map)."""
    from loongforge_b200.models.registry import get_model_config
    from tools.convert_checkpoint import name_maps as nm
    from tools.convert_checkpoint.convert import load_hf

    cfg = get_model_config(model_name, **(overrides or {}))
    cfg.pad_vocab(1)
    margs = {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in vars(cfg).items()}
    dims = _dims(margs)
    mc = nm.hf_to_mcore(load_hf(hf_dir), nm.FAMILIES[family], padded_vocab=cfg.padded_vocab_size, **dims)
    write_model_tensors(ckpt_root, mc, margs)
    return len(mc)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--to", required=True, choices=["hf", "dist"])
    ap.add_argument("--load", required=True)
    ap.add_argument("--save", required=True)
    ap.add_argument("--family", default="llama3", help="name map of tools/convert_checkpoint/name_maps.py")
    ap.add_argument("--model-name", default=None, help="architecture preset (needed for --to dist)")
    ap.add_argument("--iteration", type=int, default=None)
    a = ap.parse_args(argv)
    if a.to == "hf":
        n = dist_to_hf(a.load, a.save, a.family, a.iteration)
    else:
        if not a.model_name:
            ap.error("--to dist needs --model-name")
        n = hf_to_dist(a.load, a.save, a.family, a.model_name)
    print(f"converted {n} tensors -> {a.save}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
