"""Release export: the model weights of a training checkpoint as ONE ``.safetensors`` (or ``.pt``) file.

    python -m loongforge_b200.embodied.export_checkpoint --ckpt RUN/checkpoints[/step_00001000] --out policy.safetensors
        [--format safetensors|pt] [--dtype bf16|fp16|fp32] [--keep-lora] [--strip-prefix policy.]

``--ckpt`` is a ``step_*`` directory or the directory holding them (then the ``latest`` marker, else the highest step, is
taken). Both checkpoint formats are read without a process group: ``model_optim.pt`` directly, a DCP directory through the
metadata-driven single-process reader. LoRA checkpoints are folded (``W + s B A``, the scale from the ``lora`` entry of
``meta.json``) unless ``--keep-lora``; optimizer state, RNG and data-loader positions stay behind. Tensors that share
storage (tied tables) are written once per name as separate copies, as the safetensors format requires.

(reference: loongforge/embodied/tools/dcp_to_safetensors.py:1-130)
"""
from __future__ import annotations

import argparse
import glob
import json
import math
import os
import tempfile
from typing import Dict, Optional

import torch

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def resolve_step_dir(path: str) -> str:
    if os.path.isfile(os.path.join(path, "meta.json")):
        return path
    marker = os.path.join(path, "latest")
    if os.path.isfile(marker):
        with open(marker) as f:
            name = f.read().strip()
        cand = os.path.join(path, name if name.startswith("step_") else f"step_{int(name):08d}")
        if os.path.isdir(cand):
            return cand
    steps = sorted(glob.glob(os.path.join(path, "step_*")))
    if not steps:
        raise FileNotFoundError(f"no checkpoint (meta.json or step_* directories) under {path}")
    return steps[-1]


def read_model_state(step_dir: str) -> Dict[str, torch.Tensor]:
    with open(os.path.join(step_dir, "meta.json")) as f:
        fmt = json.load(f).get("format", "pt")
    if fmt == "dcp":
        from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

        with tempfile.TemporaryDirectory() as tmp:
            flat = os.path.join(tmp, "flat.pt")
            dcp_to_torch_save(os.path.join(step_dir, "dcp"), flat)
            blob = torch.load(flat, map_location="cpu", weights_only=False)
    else:
        blob = torch.load(os.path.join(step_dir, "model_optim.pt"), map_location="cpu", weights_only=False)
    return blob["model"] if isinstance(blob, dict) and "model" in blob else blob


def fold_lora(state: Dict[str, torch.Tensor], lora: dict) -> Dict[str, torch.Tensor]:
    """``X.base.weight`` + ``X.lora_a.weight`` + ``X.lora_b.weight`` -> ``X.weight`` (and ``X.base.bias`` -> ``X.bias``)."""
    rank, alpha = int(lora["rank"]), float(lora["alpha"])
    scale = alpha / math.sqrt(rank) if lora.get("use_rslora") else alpha / rank
    out: Dict[str, torch.Tensor] = {}
    for name, t in state.items():
        if ".lora_a." in name or ".lora_b." in name:
            continue
        if name.endswith(".base.weight"):
            stem = name[:-len(".base.weight")]
            a, b = state[stem + ".lora_a.weight"], state[stem + ".lora_b.weight"]
            out[stem + ".weight"] = (t.float() + scale * (b.float() @ a.float())).to(t.dtype)
        elif name.endswith(".base.bias"):
            out[name[:-len(".base.bias")] + ".bias"] = t
        else:
            out[name] = t
    return out


def export(ckpt: str, out: str, fmt: str = "safetensors", dtype: Optional[str] = None, keep_lora: bool = False,
           strip_prefix: str = "") -> Dict[str, object]:
    step_dir = resolve_step_dir(ckpt)
    with open(os.path.join(step_dir, "meta.json")) as f:
        meta = json.load(f)
    state = {k: v for k, v in read_model_state(step_dir).items() if isinstance(v, torch.Tensor)}
    folded = 0
    if meta.get("lora") and not keep_lora:
        before = len(state)
        state = fold_lora(state, meta["lora"])
        folded = (before - len(state)) // 2
    if strip_prefix:
        state = {(k[len(strip_prefix):] if k.startswith(strip_prefix) else k): v for k, v in state.items()}
    if dtype:
        state = {k: (v.to(DTYPES[dtype]) if v.is_floating_point() else v) for k, v in state.items()}
    state = {k: v.detach().contiguous().clone() for k, v in state.items()}   # no shared storage between names
    os.makedirs(os.path.dirname(os.path.abspath(out)) or ".", exist_ok=True)
    if fmt == "safetensors":
        from safetensors.torch import save_file
        save_file(state, out, metadata={"step": str(meta.get("step")), "format": "pt"})
    else:
        torch.save(state, out)
    return {"step_dir": step_dir, "tensors": len(state), "lora_folded": folded,
            "bytes": sum(v.numel() * v.element_size() for v in state.values())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="export the model weights of an embodied training checkpoint to one file")
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--format", choices=["safetensors", "pt"], default="safetensors")
    ap.add_argument("--dtype", choices=sorted(DTYPES), default=None)
    ap.add_argument("--keep-lora", action="store_true")
    ap.add_argument("--strip-prefix", default="")
    a = ap.parse_args(argv)
    info = export(a.ckpt, a.out, a.format, a.dtype, a.keep_lora, a.strip_prefix)
    print(f"{info['step_dir']} -> {a.out}: {info['tensors']} tensors, {info['bytes'] / 2**20:.1f} MiB"
          + (f", {info['lora_folded']} LoRA layers folded" if info["lora_folded"] else ""))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
