"""Checkpoint save / load in the Megatron ``torch_dist`` layout and in the legacy per-rank layout.

Directory layout written here (loongforge/train/checkpointing.py:157-224,302-354 and the
``torch_dist`` strategy the reference inherits from Megatron):

    <dir>/latest_checkpointed_iteration.txt        integer iteration, or ``release``
    <dir>/iter_0000020/metadata.json               {"sharded_backend": "torch_dist", ...}
    <dir>/iter_0000020/common.pt                   non-tensor state (args, iteration, scheduler, ...)
    <dir>/iter_0000020/.metadata                   torch.distributed.checkpoint global index
    <dir>/iter_0000020/__{rank}_{k}.distcp         this rank's tensor shards

Model tensors are stored under their Megatron module paths with GLOBAL (unsharded) shapes and
per-shard offsets, so a checkpoint can be loaded with a different TP/PP/DP layout. SwiGLU FC1
(``[gate; up]``) is stored as two shards per rank. Optimizer state (fp32 master weights and
both Adam moments) is stored as flat 1-D tensors per (parameter, model-parallel coordinate),
chunked by data-parallel ownership: re-shardable over DP, tied to TP/PP like the reference's
default ``dp_reshardable`` type (checkpointing.py:563-605). RNG state is one object per rank.

Legacy layout: ``iter_{:07d}/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt`` with keys
``model``, ``optimizer``, ``opt_param_scheduler``, ``rng_state``, ``iteration``,
``checkpoint_version`` (3.0), ``args``.
"""
from __future__ import annotations

import io
import json
import os
import random
import socket
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed._shard.sharded_tensor import Shard, ShardedTensor, ShardMetadata
from torch.distributed._shard.sharded_tensor.metadata import ShardedTensorMetadata, TensorProperties

from ..parallel import state as ps

TRACKER = "latest_checkpointed_iteration.txt"
CHECKPOINT_VERSION = 3.0


# ----------------------------------------------------------------------------- naming
def iteration_dir(root: str, iteration, release: bool = False) -> str:
    return os.path.join(root, "release" if release else "iter_{:07d}".format(iteration))


def legacy_rank_dir(root: str, iteration, tp_rank: int, pp_rank: int, pp_size: int, ep_rank: int = 0,
                    ep_size: int = 1, release: bool = False) -> str:
    name = "mp_rank_{:02d}".format(tp_rank)
    if pp_size > 1:
        name += "_{:03d}".format(pp_rank)
    if ep_size > 1:
        name += "_{:03d}".format(ep_rank)
    return os.path.join(iteration_dir(root, iteration, release), name)


def read_tracker(root: str) -> Tuple[Optional[int], bool]:
    p = os.path.join(root, TRACKER)
    if not os.path.isfile(p):
        return None, False
    s = open(p).read().strip()
    if s == "release":
        return 0, True
    return int(s), False


def write_tracker(root: str, iteration, release: bool = False) -> None:
    with open(os.path.join(root, TRACKER), "w") as f:
        f.write("release" if release else str(iteration))


# ----------------------------------------------------------------------------- process group bootstrap
def _ensure_pg():
    if dist.is_initialized():
        return
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)


# ----------------------------------------------------------------------------- sharded tensors
def _placement(rank: int, t: torch.Tensor) -> str:
    return f"rank:{rank}/{'cuda:' + str(t.device.index) if t.is_cuda else 'cpu'}"


def _props(t: torch.Tensor) -> TensorProperties:
    return TensorProperties(dtype=t.dtype, layout=torch.strided, requires_grad=False,
                            memory_format=torch.contiguous_format, pin_memory=False)


def _param_tp(p: torch.Tensor, st) -> Tuple[int, int]:
    """(rank, size) of the tensor-parallel sharding of THIS parameter: the owning module's own degree when it recorded
    one (expert tensor parallelism, encoders with their own TP degree), else the job's main TP."""
    if hasattr(p, "tp_shards"):
        return p.tp_shard_rank, p.tp_shards
    if getattr(p, "is_expert", False):
        return st.etp_rank, st.dims.etp
    return st.tp_rank, st.dims.tp


def param_global_layout(p: torch.Tensor, tp_rank: int, tp_size: int):
    """[(global_offsets, local_slice)] pieces of parameter `p` in its unsharded tensor, and the global shape."""
    shape = list(p.shape)
    dim = getattr(p, "partition_dim", -1)
    if not getattr(p, "tensor_model_parallel", False) or dim < 0 or tp_size == 1:
        return [([0] * p.dim(), tuple(slice(None) for _ in shape))], shape
    stride = getattr(p, "partition_stride", 1)
    gshape = list(shape)
    gshape[dim] = shape[dim] * tp_size
    pieces = []
    blk_local = shape[dim] // stride
    blk_global = gshape[dim] // stride
    for b in range(stride):
        off = [0] * p.dim()
        off[dim] = b * blk_global + tp_rank * blk_local
        sl = [slice(None)] * p.dim()
        sl[dim] = slice(b * blk_local, (b + 1) * blk_local)
        pieces.append((off, tuple(sl)))
    return pieces, gshape


def _complement_chunks(gshape, dim, taken: List[Tuple[int, int]]):
    """Intervals of [0, gshape[dim]) not covered by `taken` (sorted, disjoint)."""
    out, cur = [], 0
    for a, b in sorted(taken):
        if a > cur:
            out.append((cur, a))
        cur = b
    if cur < gshape[dim]:
        out.append((cur, gshape[dim]))
    return out


def make_sharded(local_pieces: List[Tuple[List[int], torch.Tensor]], gshape, rank: int,
                 all_pieces: Optional[List[Tuple[int, List[int], List[int]]]] = None) -> ShardedTensor:
    """ShardedTensor from this rank's pieces. `all_pieces` = [(owner_rank, offsets, sizes)] over ALL
    ranks (needed for a collective save); when None, fake complementary entries owned by a
    virtual peer complete the cover (enough for an independent, per-rank load)."""
    ref = local_pieces[0][1] if local_pieces else None
    metas = []
    if all_pieces is not None:
        for owner, off, sizes in all_pieces:
            metas.append(ShardMetadata(shard_offsets=list(off), shard_sizes=list(sizes),
                                       placement=f"rank:{owner}/cpu"))
    else:
        dim = 0
        for d in range(len(gshape)):
            if any(t.shape[d] != gshape[d] for _, t in local_pieces):
                dim = d
        taken = []
        for off, t in local_pieces:
            metas.append(ShardMetadata(shard_offsets=list(off), shard_sizes=list(t.shape), placement=f"rank:{rank}/cpu"))
            taken.append((off[dim], off[dim] + t.shape[dim]))
        world = dist.get_world_size()
        other = (rank + 1) % world
        comp = _complement_chunks(gshape, dim, taken)
        assert not comp or world > 1, "a single process must hold the whole tensor"
        for a, b in comp:
            off = [0] * len(gshape)
            off[dim] = a
            sz = list(gshape)
            sz[dim] = b - a
            metas.append(ShardMetadata(shard_offsets=off, shard_sizes=sz, placement=f"rank:{other}/cpu"))
    props = _props(ref) if ref is not None else TensorProperties(dtype=torch.float32)
    stm = ShardedTensorMetadata(shards_metadata=metas, size=torch.Size(gshape), tensor_properties=props)
    mine = {(tuple(m.shard_offsets), tuple(m.shard_sizes)): m for m in metas if m.placement.rank() == rank}
    shards = [Shard(t, mine[(tuple(off), tuple(t.shape))]) for off, t in local_pieces]
    return ShardedTensor._init_from_local_shards_and_global_metadata(shards, stm)


# ----------------------------------------------------------------------------- model keys
def model_param_items(trainer):
    """Yield (global_key, param) for every parameter of every local model chunk, with layer
    indices translated from stage-local to global numbering."""
    for chunk in trainer.models:
        mod = chunk.module
        layer_numbers = getattr(mod.decoder, "layer_numbers", None) if hasattr(mod, "decoder") else None
        for name, p in mod.named_parameters():
            key = name
            # stage-local layer index -> global one; the language model may sit under a prefix ("foundation_model."
            # in vision-language models), the encoder's own "...image_encoder.decoder.layers." is never pipelined
            at = name.find("decoder.layers.")
            if layer_numbers is not None and at >= 0 and "encoder" not in name[:at]:
                head, rest = name[:at + len("decoder.layers.")], name[at + len("decoder.layers."):]
                idx, _, tail = rest.partition(".")
                key = f"{head}{layer_numbers[int(idx)]}.{tail}"
            ge = getattr(p, "expert_global_index", None)
            if ge is not None:  # "...linear_fc1.weight{local}" -> "...linear_fc1.weight{global}" under expert parallelism
                key = key[:key.rindex("weight")] + f"weight{ge}"
            yield key, p


def _gather_obj(obj):
    if dist.get_world_size() == 1:
        return [obj]
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def build_save_state(trainer, stage: bool = False) -> Dict[str, object]:
    """``stage``: every tensor is a private host copy, so the state stays valid while training goes on (asynchronous save)."""
    st = trainer.st
    own = (lambda t: t.to("cpu", copy=True)) if stage else (lambda t: t.contiguous())
    rank = dist.get_rank()
    tp, tpr = st.dims.tp, st.tp_rank
    # ---- who owns what (model replicas: the first data-parallel rank writes)
    local_desc = []  # (key, gshape, [(offsets, sizes)]), only from writers
    local_tensors: Dict[str, List[Tuple[List[int], torch.Tensor]]] = {}
    gshapes = {}
    dp_writer = st.rank_in("dp_cp") == 0
    for key, p in model_param_items(trainer):
        is_expert = getattr(p, "is_expert", False)
        writer = (st.edp_rank == 0) if is_expert else dp_writer
        p_rank, p_size = _param_tp(p, st)
        pieces, gshape = param_global_layout(p, p_rank, p_size)
        gshapes[key] = gshape
        dup = not getattr(p, "tensor_model_parallel", False)
        # replicas beyond the tensor's own sharding degree do not write (a TP-1 encoder beside a TP-2 decoder)
        if not writer or (st.etp_rank if is_expert else tpr) >= (1 if dup else p_size):
            continue
        if getattr(p, "shared_embedding_replica", False):
            continue
        data = p.detach()
        local_tensors[key] = [(off, own(data[sl])) for off, sl in pieces]
        local_desc.append((key, gshape, [(off, list(t.shape)) for off, t in local_tensors[key]]))
    # ---- optimizer: flat chunks per (param, model-parallel coordinate)
    opt_local: Dict[str, List[Tuple[List[int], torch.Tensor]]] = {}
    opt_desc = []
    key_of = {id(p): key for key, p in model_param_items(trainer)}
    coord = f"tp{tpr}of{tp}.ep{st.ep_rank}of{st.dims.ep}"
    sharded = trainer.optimizer.sharded
    save_optim = not getattr(trainer.tcfg, "no_save_optim", False)
    for name, pieces in (trainer.optimizer.sharded_state().items() if save_optim else ()):
        if not sharded and st.rank_in("dp_cp") != 0:
            continue
        for piece in pieces:
            if getattr(piece["param"], "shared_embedding_replica", False):
                continue  # the first pipeline stage writes the shared word embedding and its optimizer state
            for kind in ("master", "exp_avg", "exp_avg_sq"):
                k = f"optimizer.state.{kind}.{key_of.get(id(piece['param']), name)}.{coord}"
                t = own(piece[kind].detach())
                opt_local.setdefault(k, []).append(([piece["offset"]], t))
                gshapes[k] = [piece["param_numel"]]
    for k, lst in opt_local.items():
        opt_desc.append((k, gshapes[k], [(off, list(t.shape)) for off, t in lst]))
    # ---- exchange descriptions so that every rank builds identical global metadata
    everyone = _gather_obj((rank, local_desc + opt_desc))
    table: Dict[str, Tuple[list, list]] = {}
    for r, descs in everyone:
        for key, gshape, pieces in descs:
            ent = table.setdefault(key, (gshape, []))
            for off, sizes in pieces:
                ent[1].append((r, off, sizes))
    state: Dict[str, object] = {}
    for key, (gshape, allp) in table.items():
        mine = local_tensors.get(key) or opt_local.get(key) or []
        # optimizer pieces of a parameter may leave gaps (alignment padding is not state): fill the cover
        if len(gshape) == 1:
            taken = sorted((off[0], off[0] + sz[0]) for _, off, sz in allp)
            for a, b in _complement_chunks(gshape, 0, taken):
                allp = allp + [(allp[0][0], [a], [b - a])]
                if allp[0][0] == rank:
                    mine = mine + [([a], torch.zeros(b - a, dtype=(mine[0][1].dtype if mine else torch.float32)))]
        state[key] = make_sharded(mine, gshape, rank, allp)
    # ---- per-rank objects
    if not getattr(trainer.tcfg, "no_save_rng", False):
        buf = io.BytesIO()
        torch.save(get_rng_state(), buf)
        state[f"rng_state/shard_{st.pp_rank}.{st.tp_rank}.{st.rank_in('dp_cp')}"] = buf
    return state


def get_rng_state() -> dict:
    s = {"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(),
         "torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        s["cuda_rng_state"] = torch.cuda.get_rng_state()
    # named streams of the model-parallel tracker (dropout inside tensor- / expert-parallel regions); reference:
    # loongforge/train/checkpointing.py:511-552 saves them as `rng_tracker_states`
    from ..parallel.random import get_rng_tracker
    s["rng_tracker_states"] = get_rng_tracker().get_states()
    return s


def set_rng_state(s: dict) -> None:
    random.setstate(s["random_rng_state"])
    np.random.set_state(s["np_rng_state"])
    torch.set_rng_state(s["torch_rng_state"])
    if torch.cuda.is_available() and "cuda_rng_state" in s:
        torch.cuda.set_rng_state(s["cuda_rng_state"])
    if s.get("rng_tracker_states"):
        from ..parallel.random import get_rng_tracker
        get_rng_tracker().set_states(s["rng_tracker_states"])


def common_state(trainer) -> dict:
    t = trainer
    return {
        "args": {"model": {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in vars(t.mcfg).items()},
                 "train": {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in vars(t.tcfg).items()},
                 "parallel": {"tp": t.st.dims.tp, "pp": t.st.dims.pp, "cp": t.st.dims.cp, "ep": t.st.dims.ep,
                              "dp": t.st.dp_size, "world": t.st.world_size}},
        "checkpoint_version": CHECKPOINT_VERSION,
        "iteration": t.iteration,
        "consumed_samples": t.consumed_samples,
        "num_floating_point_operations_so_far": t.num_flops_so_far,
        "opt_param_scheduler": t.scheduler.state_dict(),
        "optimizer": t.optimizer.state_dict(),
    }


# ----------------------------------------------------------------------------- save / load (torch_dist)
def finalize_async_save(trainer) -> None:
    """Waits for the checkpoint write started by an asynchronous save and only then publishes it in the tracker
    file, so that a crash during the write never leaves the tracker pointing at a partial checkpoint."""
    pending = getattr(trainer, "_pending_save", None)
    if pending is None:
        return
    fut, root, iteration, release = pending
    fut.result()
    trainer._pending_save = None
    if dist.get_world_size() > 1:
        dist.barrier()
    if dist.get_rank() == 0:
        write_tracker(root, iteration, release)
    if dist.get_world_size() > 1:
        dist.barrier()


def save_checkpoint(root: str, trainer, *, fmt: Optional[str] = None, release: bool = False,
                    async_save: Optional[bool] = None) -> str:
    fmt = fmt or trainer.tcfg.ckpt_format
    if fmt == "torch":
        return save_legacy(root, trainer, release=release)
    _ensure_pg()
    finalize_async_save(trainer)  # at most one write in flight
    if async_save is None:
        async_save = bool(getattr(trainer.tcfg, "async_save", False))
    d = iteration_dir(root, trainer.iteration, release)
    rank = dist.get_rank()
    if rank == 0:
        os.makedirs(d, exist_ok=True)
    if dist.get_world_size() > 1:
        dist.barrier()
    state = build_save_state(trainer, stage=async_save)
    fut = None
    if async_save:
        # the write (and its metadata collectives) runs on a worker thread over a process group of its own, so it
        # cannot interleave with the training collectives; the tensors were copied to host memory above
        import concurrent.futures
        if getattr(trainer, "_ckpt_pg", None) is None:
            trainer._ckpt_pg = dist.new_group(backend="gloo")
            trainer._ckpt_pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
        fut = trainer._ckpt_pool.submit(dcp.save, state, checkpoint_id=d, process_group=trainer._ckpt_pg)
    else:
        dcp.save(state, checkpoint_id=d)
    if rank == 0:
        torch.save(common_state(trainer), os.path.join(d, "common.pt"))
        with open(os.path.join(d, "metadata.json"), "w") as f:
            json.dump({"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
                       "common_backend_version": 1}, f)
        if fut is None:
            write_tracker(root, trainer.iteration, release)
    if fut is not None:
        trainer._pending_save = (fut, root, trainer.iteration, release)
        return d
    if dist.get_world_size() > 1:
        dist.barrier()
    return d


def load_checkpoint(root: str, trainer, *, load_optim: bool = True, load_rng: bool = True,
                    iteration: Optional[int] = None, strict: bool = True) -> int:
    """Restores model (any TP/PP/DP layout), and optimizer / scheduler / RNG when the layout
    allows (same TP/PP for the optimizer; same world layout for RNG). Returns the iteration."""
    it, release = (iteration, False) if iteration is not None else read_tracker(root)
    if it is None:
        return 0
    d = iteration_dir(root, it, release)
    if not os.path.isfile(os.path.join(d, "metadata.json")):
        return load_legacy(root, trainer, it, release, load_optim=load_optim, load_rng=load_rng)
    _ensure_pg()
    st = trainer.st
    rank = dist.get_rank()
    common = torch.load(os.path.join(d, "common.pt"), weights_only=False)
    saved_par = common["args"]["parallel"]
    same_mp = saved_par["tp"] == st.dims.tp and saved_par["pp"] == st.dims.pp and saved_par["ep"] == st.dims.ep
    same_world = same_mp and saved_par["dp"] == st.dp_size and saved_par["cp"] == st.dims.cp
    tp, tpr = st.dims.tp, st.tp_rank
    state: Dict[str, object] = {}
    targets = []
    for key, p in model_param_items(trainer):
        is_expert = getattr(p, "is_expert", False)
        pieces, gshape = param_global_layout(p, *_param_tp(p, st))
        bufs = [(off, torch.empty_like(p.detach()[sl], device="cpu").contiguous()) for off, sl in pieces]
        state[key] = make_sharded(bufs, gshape, rank)
        targets.append((p, pieces, bufs))
    opt_targets = []
    if load_optim and same_mp:
        coord = f"tp{tpr}of{tp}.ep{st.ep_rank}of{st.dims.ep}"
        key_of = {id(p): k for k, p in model_param_items(trainer)}
        for name, pieces in trainer.optimizer.sharded_state().items():
            for piece in pieces:
                for kind in ("master", "exp_avg", "exp_avg_sq"):
                    k = f"optimizer.state.{kind}.{key_of.get(id(piece['param']), name)}.{coord}"
                    buf = torch.empty(piece["numel"], dtype=piece[kind].dtype)
                    state.setdefault(k + f"@{piece['offset']}", None)
                    opt_targets.append((k, piece, kind, buf))
        # one ShardedTensor per key holding all of this rank's pieces
        by_key: Dict[str, list] = {}
        for k, piece, kind, buf in opt_targets:
            by_key.setdefault(k, []).append(([piece["offset"]], buf, piece["param_numel"]))
        for k in [k for k in state if "@" in k]:
            del state[k]
        for k, lst in by_key.items():
            state[k] = make_sharded([(o, b) for o, b, _ in lst], [lst[0][2]], rank)
    rng_key = f"rng_state/shard_{st.pp_rank}.{st.tp_rank}.{st.rank_in('dp_cp')}"
    if load_rng and same_world:
        state[rng_key] = io.BytesIO()
    dcp.load(state, checkpoint_id=d, no_dist=True)
    with torch.no_grad():
        for p, pieces, bufs in targets:
            for (off, sl), (_, b) in zip(pieces, bufs):
                p.data[sl].copy_(b)
    if load_optim and same_mp:
        for k, piece, kind, buf in opt_targets:
            if kind == "master":
                piece["set_master"](buf)
            else:
                piece[kind].copy_(buf)
        trainer.optimizer.load_state_dict(common["optimizer"])
        trainer.scheduler.load_state_dict(common["opt_param_scheduler"])
    else:
        trainer.optimizer.reload_model_params()
    if load_rng and same_world:
        state[rng_key].seek(0)
        set_rng_state(torch.load(state[rng_key], weights_only=False))
    trainer.iteration = common["iteration"]
    trainer.consumed_samples = common.get("consumed_samples", 0)
    trainer.num_flops_so_far = common.get("num_floating_point_operations_so_far", 0.0)
    if dist.get_world_size() > 1:
        dist.barrier()
    return trainer.iteration


def _named_params(trainer):
    for chunk in trainer.models:
        for name, p in chunk.module.named_parameters():
            yield name, p


# ----------------------------------------------------------------------------- legacy format
def save_legacy(root: str, trainer, *, release: bool = False) -> str:
    st = trainer.st
    d = legacy_rank_dir(root, trainer.iteration, st.tp_rank, st.pp_rank, st.dims.pp, st.ep_rank, st.dims.ep, release)
    if st.rank_in("dp_cp") == 0:
        os.makedirs(d, exist_ok=True)
        sd = common_state(trainer)
        if len(trainer.models) == 1:
            sd["model"] = {k: v.detach().cpu() for k, v in trainer.models[0].module.state_dict().items()}
        else:
            for i, m in enumerate(trainer.models):
                sd[f"model{i}"] = {k: v.detach().cpu() for k, v in m.module.state_dict().items()}
        sd["rng_state"] = [get_rng_state()]
        torch.save(sd, os.path.join(d, "model_optim_rng.pt"))
    # optimizer shards of every data-parallel rank
    od = os.path.join(d, f"distrib_optim_dp{st.rank_in('dp_cp'):03d}.pt")
    os.makedirs(d, exist_ok=True)
    torch.save({n: [{k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in pc.items() if k not in ("set_master", "param")}
                    for pc in pcs]
                for n, pcs in trainer.optimizer.sharded_state().items()}, od)
    if dist.is_initialized():
        dist.barrier()
    if (not dist.is_initialized()) or dist.get_rank() == 0:
        write_tracker(root, trainer.iteration, release)
    return d


def load_legacy(root: str, trainer, it: int, release: bool, *, load_optim: bool = True, load_rng: bool = True) -> int:
    st = trainer.st
    d = legacy_rank_dir(root, it, st.tp_rank, st.pp_rank, st.dims.pp, st.ep_rank, st.dims.ep, release)
    sd = torch.load(os.path.join(d, "model_optim_rng.pt"), weights_only=False, map_location="cpu")
    if len(trainer.models) == 1:
        trainer.models[0].module.load_state_dict(sd["model"], strict=False)
    else:
        for i, m in enumerate(trainer.models):
            m.module.load_state_dict(sd[f"model{i}"], strict=False)
    od = os.path.join(d, f"distrib_optim_dp{st.rank_in('dp_cp'):03d}.pt")
    if load_optim and os.path.isfile(od) and "optimizer" in sd:
        saved = torch.load(od, weights_only=False, map_location="cpu")
        cur = trainer.optimizer.sharded_state()
        for name, pieces in cur.items():
            for pc, sv in zip(pieces, saved.get(name, [])):
                pc["set_master"](sv["master"])
                for kind in ("exp_avg", "exp_avg_sq"):
                    pc[kind].copy_(sv[kind])
        trainer.optimizer.load_state_dict(sd["optimizer"])
        trainer.scheduler.load_state_dict(sd["opt_param_scheduler"])
    else:
        trainer.optimizer.reload_model_params()
    if load_rng and sd.get("rng_state"):
        set_rng_state(sd["rng_state"][0])
    trainer.iteration = sd.get("iteration", it)
    trainer.consumed_samples = sd.get("consumed_samples", 0)
    return trainer.iteration
