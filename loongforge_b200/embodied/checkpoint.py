"""Checkpointing of the embodied stack: single-file ``.pt`` and torch DCP directory formats, per-rank RNG and
data-loader state, ZeRO optimizer consolidation, LoRA adapter metadata, ``latest`` tracker and resume, and a DCP ->
single-file export (reference: loongforge/embodied/distributed/checkpoint.py:71-975, tools/dcp_to_safetensors.py)."""
from __future__ import annotations

import glob
import json
import os
import random
from typing import Any, Dict, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn


def _unwrap(model: nn.Module) -> nn.Module:
    return model.module if isinstance(model, nn.parallel.DistributedDataParallel) else model


def rng_state() -> Dict[str, Any]:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def set_rng_state(st: Dict[str, Any]) -> None:
    random.setstate(st["python"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])


def _step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"step_{step:08d}")


def latest_step(root: str) -> Optional[int]:
    p = os.path.join(root, "latest")
    if not os.path.isfile(p):
        return None
    with open(p) as f:
        return int(f.read().strip())


def save_checkpoint(root: str, step: int, model: nn.Module, optimizer, scheduler=None, *, fmt: str = "pt",
                    dataloader_state: Optional[dict] = None, lora_meta: Optional[dict] = None, rank: int = 0,
                    world: int = 1, async_save: bool = False) -> str:
    """``optimizer=None`` stores the weights only. ``async_save`` (pt format): tensors are copied to the host here and the
    file is written by a background thread (``wait_async_saves`` joins them; the ``latest`` marker moves only when the
    file is complete)."""
    d = _step_dir(root, step)
    os.makedirs(d, exist_ok=True)
    inner = _unwrap(model)
    if fmt == "dcp":
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import get_state_dict

        if optimizer is None:
            from torch.distributed.checkpoint.state_dict import get_model_state_dict
            dcp.save({"model": get_model_state_dict(inner)}, checkpoint_id=os.path.join(d, "dcp"))
        else:
            msd, osd = get_state_dict(inner, optimizer)
            dcp.save({"model": msd, "optim": osd}, checkpoint_id=os.path.join(d, "dcp"))
    else:
        sharded = hasattr(optimizer, "local_state_dict")  # ZeRO-1: every rank writes the shard it owns, keyed by name
        if sharded:
            torch.save(optimizer.local_state_dict(), os.path.join(d, f"optim_shard_{rank:05d}.pt"))
        if rank == 0:
            blob = {"model": inner.state_dict(), "optim": None if (sharded or optimizer is None) else optimizer.state_dict()}
            target = os.path.join(d, "model_optim.pt")
            if async_save:
                blob = _to_host(blob)
                import threading
                th = threading.Thread(target=_write_then_mark, args=(blob, target, root, step), daemon=False)
                th.start()
                _PENDING.append(th)
            else:
                torch.save(blob, target)
    # per-rank auxiliary state
    torch.save({"rng": rng_state(), "dataloader": dataloader_state}, os.path.join(d, f"aux_rank{rank:05d}.pt"))
    if rank == 0:
        meta = {"step": step, "format": fmt, "world_size": world,
                "scheduler": scheduler.state_dict() if scheduler is not None else None, "lora": lora_meta}
        with open(os.path.join(d, "meta.json"), "w") as f:
            json.dump(meta, f)
    if world > 1 and dist.is_initialized():
        dist.barrier()
    if rank == 0 and not (async_save and fmt != "dcp"):
        _mark_latest(root, step)
    return d


_PENDING: list = []


def _mark_latest(root: str, step: int) -> None:
    tmp = os.path.join(root, "latest.tmp")
    with open(tmp, "w") as f:
        f.write(str(step))
    os.replace(tmp, os.path.join(root, "latest"))


def _to_host(obj):
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_host(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_host(v) for v in obj)
    return obj


def _write_then_mark(blob, target: str, root: str, step: int) -> None:
    torch.save(blob, target + ".tmp")
    os.replace(target + ".tmp", target)
    _mark_latest(root, step)


def wait_async_saves() -> None:
    while _PENDING:
        _PENDING.pop().join()


def load_checkpoint(root: str, model: nn.Module, optimizer=None, scheduler=None, *, step: Optional[int] = None,
                    rank: int = 0, restore_rng: bool = True) -> Optional[dict]:
    step = latest_step(root) if step is None else step
    if step is None:
        return None
    d = _step_dir(root, step)
    with open(os.path.join(d, "meta.json")) as f:
        meta = json.load(f)
    inner = _unwrap(model)
    if meta["format"] == "dcp":
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import get_state_dict, set_state_dict

        msd, osd = get_state_dict(inner, optimizer) if optimizer is not None else (inner.state_dict(), {})
        state = {"model": msd, "optim": osd} if optimizer is not None else {"model": msd}
        dcp.load(state, checkpoint_id=os.path.join(d, "dcp"))
        if optimizer is not None:
            set_state_dict(inner, optimizer, model_state_dict=state["model"], optim_state_dict=state["optim"])
        else:
            inner.load_state_dict(state["model"])
    else:
        blob = torch.load(os.path.join(d, "model_optim.pt"), map_location="cpu", weights_only=False)
        inner.load_state_dict(blob["model"])
        if optimizer is not None:
            shards = sorted(glob.glob(os.path.join(d, "optim_shard_*.pt")))
            if shards and hasattr(optimizer, "load_local_state_dicts"):
                # any number of shard files (the world size at save time) into the present partition
                optimizer.load_local_state_dicts([torch.load(f, map_location="cpu", weights_only=False) for f in shards])
            elif shards:
                merged = {}
                for f in shards:
                    merged.update(torch.load(f, map_location="cpu", weights_only=False)["state"])
                raise ValueError(f"{d} holds a sharded (zero1) optimizer state of {len(merged)} tensors; resume with strategy=zero1")
            elif blob["optim"] is not None:
                optimizer.load_state_dict(blob["optim"])
    if scheduler is not None and meta.get("scheduler"):
        scheduler.load_state_dict(meta["scheduler"])
    aux_path = os.path.join(d, f"aux_rank{rank:05d}.pt")
    aux = torch.load(aux_path, map_location="cpu", weights_only=False) if os.path.isfile(aux_path) else {}
    if restore_rng and aux.get("rng"):
        set_rng_state(aux["rng"])
    return {"step": meta["step"], "dataloader": aux.get("dataloader"), "lora": meta.get("lora")}


def dcp_to_single_file(dcp_dir: str, out_path: str) -> None:
    """Export the model weights of a DCP checkpoint to one ``torch.save`` file (no process group needed)."""
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

    dcp_to_torch_save(dcp_dir, out_path)
