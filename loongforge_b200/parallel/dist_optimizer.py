"""Sharded (ZeRO-1 style) AdamW over the flat buffers of ``parallel/ddp.py``.

Each data-parallel rank owns one contiguous shard of every bucket: it keeps the fp32 master
weights and both Adam moments for that shard only, updates them from the reduce-scattered
gradient shard with ONE fused kernel launch per bucket (which also writes the bf16 model
weights back into the parameter buffer) and all-gathers the parameter bucket. This is the
behaviour the reference gets from Megatron's ``DistributedOptimizer`` with
``--use-distributed-optimizer`` (loongforge/train/training_utils.py:1073-1084), including bf16
moments (patches/TransformerEngine_v2.9/.../fused_adam.py.patch:18-350, described in
docs/source/features/optimizer_support.md:54-73).

With ``use_distributed_optimizer=False`` every rank keeps full state (plain DDP + Adam).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from . import state as ps
from .ddp import Bucket, DistributedDataParallel, ParamAndGradBuffer


@dataclasses.dataclass
class OptimizerConfig:
    lr: float = 1e-4
    min_lr: float = 0.0
    weight_decay: float = 0.01
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    exp_avg_dtype: torch.dtype = torch.float32
    exp_avg_sq_dtype: torch.dtype = torch.float32
    overlap_param_gather: bool = False
    # keep the fp32 master of bf16 parameters as (bf16 weight in the parameter buffer, int16 remainder):
    # exact, and 2 bytes per parameter less optimizer memory
    master_as_remainder: bool = False
    # fp32 masters and Adam moments in pinned host memory, updated by the native host AdamW; per step the gradient
    # shard goes device -> host and the refreshed weights host -> device on a side stream
    cpu_offload: bool = False
    # part of the optimizer state (by elements, whole shards) that lives on the host when cpu_offload is on
    # (reference: --optimizer-offload-fraction, docs/source/features/optimizer_support.md)
    offload_fraction: float = 1.0
    optimizer: str = "adam"  # "adam" (AdamW) or "sgd" (momentum in the first-moment buffer)
    sgd_momentum: float = 0.9
    no_weight_decay_cond: Optional[object] = None  # callable(name, param) -> bool


class _ShardState:
    """Optimizer state of one bucket shard, split into segments that share a weight decay."""

    def __init__(self, buf: ParamAndGradBuffer, b: Bucket, s: int, e: int, cfg: OptimizerConfig, sharded: bool,
                 offload: Optional[bool] = None):
        self.buf, self.bucket, self.start, self.end = buf, b, s, e
        dev = buf.param_data.device
        n = e - s
        self.offload = cfg.cpu_offload if offload is None else offload
        self.remainder = cfg.master_as_remainder and buf.param_data.dtype == torch.bfloat16 and not self.offload
        if self.offload:
            pin = dev.type == "cuda"
            host = lambda dt, fill=None: (torch.zeros if fill == 0 else torch.empty)(n, dtype=dt, pin_memory=pin)  # noqa: E731
            self._master = host(torch.float32)
            self._master.copy_(buf.param_data[s:e].float())
            self.exp_avg, self.exp_avg_sq = host(torch.float32, 0), host(torch.float32, 0)
            self.host_grad = host(torch.float32 if buf.grad_data.dtype == torch.float32 else torch.bfloat16)
            self.host_out = host(torch.bfloat16) if buf.param_data.dtype == torch.bfloat16 else None
            self.grad_event = None
        elif self.remainder:
            self.lo = torch.zeros(n, dtype=torch.int16, device=dev)  # master == bf16 weight exactly at start
            self._master = None
        else:
            self._master = buf.param_data[s:e].float().clone()
        if not self.offload:
            self.exp_avg = torch.zeros(n, dtype=cfg.exp_avg_dtype, device=dev)
            self.exp_avg_sq = torch.zeros(n, dtype=cfg.exp_avg_sq_dtype, device=dev)
        # segments: (lo, hi, weight_decay_on, tp_duplicated, name)
        self.segments = []
        for p in b.params:
            ps_, pe, _ = buf.param_index[p]
            lo, hi = max(ps_, s), min(pe, e)
            if lo >= hi:
                continue
            name = buf.named.get(p, "")
            no_wd = (cfg.no_weight_decay_cond(name, p) if cfg.no_weight_decay_cond
                     else (p.dim() == 1 or name.endswith(".bias")))
            dup = not getattr(p, "tensor_model_parallel", False)
            self.segments.append((lo - s, hi - s, not no_wd, dup, name, p, ps_))
        self.segments.sort(key=lambda t: t[0])

    @property
    def master(self) -> torch.Tensor:
        """fp32 master weights of the shard (materialised on demand in remainder mode)."""
        if self.remainder:
            return OF.master_join(self.buf.param_data[self.start:self.end], self.lo)
        return self._master

    def set_master(self, lo: int, hi: int, values: torch.Tensor) -> None:
        if self.remainder:
            w = self.buf.param_data[self.start + lo:self.start + hi]
            OF.master_split(values.float().contiguous().to(w.device), w, self.lo[lo:hi], True)
        else:
            self._master[lo:hi].copy_(values)


class DistributedOptimizer:
    def __init__(self, ddp_models: List[DistributedDataParallel], cfg: OptimizerConfig,
                 parallel_state: Optional[str] = None):
        self.models = ddp_models
        self.cfg = cfg
        self.state = ps.get_state(parallel_state)
        self.sharded = ddp_models[0].cfg.use_distributed_optimizer
        self.shards: List[_ShardState] = []
        if cfg.optimizer not in ("adam", "sgd"):
            raise ValueError(f"unknown optimizer {cfg.optimizer!r}: adam or sgd")
        if cfg.optimizer == "sgd" and (cfg.cpu_offload or cfg.master_as_remainder):
            raise ValueError("sgd runs with device-resident fp32 master weights (no offload, no remainder masters)")
        ranges = []
        for mi, m in enumerate(ddp_models):
            for buf in m._all_buffers:
                for b in buf.buckets:
                    s, e = buf.shard_range(b) if self.sharded else (b.start, b.end)
                    ranges.append((mi, buf, b, s, e))
        # shards go to the host in order until the requested fraction of the elements is reached
        budget = cfg.offload_fraction * sum(e - s for *_, s, e in ranges) if cfg.cpu_offload else 0.0
        moved = 0
        for mi, buf, b, s, e in ranges:
            off = cfg.cpu_offload and moved < budget
            moved += (e - s) if off else 0
            self.shards.append(_ShardState(buf, b, s, e, cfg, self.sharded, offload=off))
            self.shards[-1].chunk = mi
        # callables run after the data-parallel gradient reduction and before the norm / update (for reductions over
        # other groups that need the final gradients, e.g. the embedding copies of the first and last pipeline stage)
        self.post_sync_hooks: List = []
        self._gather_stream = None          # --overlap-param-gather: stream, events per (buffer, bucket), hook state
        self._gather_events: Dict[tuple, object] = {}
        self._param_bucket: Dict[int, tuple] = {}
        self._gather_hooks_installed = False
        self.step_count = 0
        self.lr = cfg.lr
        self.weight_decay = cfg.weight_decay
        self.param_groups = [{"lr": cfg.lr, "weight_decay": cfg.weight_decay}]  # scheduler-facing view
        self._gather_stream = None
        self._offload_stream = None

    # ------------------------------------------------------------------ grad norm / clipping
    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of all gradients (each logical element counted once)."""
        st = self.state
        dev = self.shards[0].exp_avg.device
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        for sh in self.shards:
            g = sh.buf.grad_data[sh.start:sh.end]
            # expert buffers are reduced over the expert-data-parallel group, which contains the TP ranks whenever experts
            # are replicated over them (ep * etp < tp * cp * dp): with a sharded optimizer every rank of that group
            # holds a DISJOINT piece, so all of them count, whatever their TP rank
            is_expert_buf = (sh.buf.dp_group is st.group("edp") and sh.buf.dp_group is not st.group("dp_cp")
                             and (st.dims.ep > 1 or (self.sharded and sh.buf.dp_size > 1)))
            # merge adjacent segments that are counted with the same multiplicity
            runs = []
            for lo, hi, _, dup, _, p, _ in sh.segments:
                # a tensor sharded `tp_shards` ways (1 = replicated) lives on that many consecutive TP ranks and is
                # repeated on the others (modules built for a parallel state with a smaller TP degree)
                copies_from = 1 if dup else getattr(p, "tp_shards", st.dims.tp)
                count = st.tp_rank < copies_from or is_expert_buf
                # the last pipeline stage's copy of the word embedding is the same logical tensor as the first stage's
                count = count and not getattr(p, "shared_embedding_replica", False)
                if not count:
                    continue
                if runs and runs[-1][1] == lo:
                    runs[-1][1] = hi
                else:
                    runs.append([lo, hi])
            for lo, hi in runs:
                OF.sum_of_squares(g[lo:hi], total)
            if not self.sharded and sh.buf.dp_size > 1:
                pass  # replicas hold identical grads; no DP reduction below for this case
        if dist.is_initialized():
            if self.sharded:
                # shards are disjoint over DP(+CP) and TP/PP ranks hold different parameters
                dist.all_reduce(total)
            else:
                g = st.group("mp")
                if g is not None:
                    dist.all_reduce(total, group=g)
        return total.sqrt()

    def _world_norm_note(self):
        return "all_reduce over WORLD is exact because every element is counted on exactly one rank"

    # ------------------------------------------------------------------ step
    # ------------------------------------------------------------------ fused step over peer memory
    def _peer_buffers(self):
        return [sh for sh in self.shards if getattr(sh.buf, "symmetric", None) is not None]

    def _peer_barrier(self, buf) -> None:
        """All ranks of the buffer's DP group reach this point (device-side epoch flags, bounded wait)."""
        from ..ops import _ext
        sym = buf.symmetric
        sym["epoch"] += 1
        C = _ext.require()
        flags = sym["block"].peer_ptrs(sym["flag_off"])
        C.peer_signal(flags, buf.dp_rank, sym["epoch"])
        C.peer_wait(flags, buf.dp_rank, sym["epoch"], _ext.status_tensor(buf.param_data.device))

    def _peer_reduce_grads(self) -> None:
        """Gradient reduce-scatter by peer loads (csrc/peer_optim.cu): after a barrier (every rank finished its
        backward) each rank pulls and sums its shard of every bucket from all DP peers, scaled by 1/dp."""
        from ..ops import _ext
        shards = list(self._peer_buffers())
        if not shards:
            return
        C = _ext.require()
        done = set()
        for sh in shards:
            if id(sh.buf) not in done:
                self._peer_barrier(sh.buf)
                done.add(id(sh.buf))
            sym = sh.buf.symmetric
            C.grad_pull_reduce(sym["block"].peer_ptrs(sym["grad_off"]), sh.buf.dp_rank, sh.start, sh.end - sh.start,
                               sh.buf.grad_scale, None)

    def _peer_adam_and_gather(self, sh, lo: int, hi: int, lr, wd, clip) -> None:
        """AdamW on [lo, hi) of the shard + parameter all-gather by peer stores, one kernel."""
        from ..ops import _ext
        cfg = self.cfg
        sym = sh.buf.symmetric
        _ext.require().adam_push(sym["block"].peer_ptrs(sym["param_off"]), sh.buf.dp_rank, sh.start + lo,
                                 sh.lo[lo:hi], sh.buf.grad_data[sh.start + lo:sh.start + hi], sh.exp_avg[lo:hi],
                                 sh.exp_avg_sq[lo:hi], lr, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, wd,
                                 self.step_count, clip)

    def _peer_ok(self, sh) -> bool:
        return (getattr(sh.buf, "symmetric", None) is not None and sh.remainder and self.sharded
                and sh.buf.grad_data.dtype == torch.float32 and sh.exp_avg.dtype == torch.float32
                and sh.exp_avg_sq.dtype == torch.float32)

    def step(self) -> tuple:
        """Finish grad sync, clip, Adam on the shards, refresh the bf16 parameters.
        Returns (update_successful, grad_norm, num_zeros)."""
        for m in self.models:
            m.finish_grad_sync()
        self.wait_param_gather()  # a bucket no forward waited for (unused parameters) must land before it is rewritten
        self._peer_reduce_grads()
        for hook in self.post_sync_hooks:
            hook()
        cfg = self.cfg
        norm = self.grad_norm()
        norm_val = float(norm.item())
        if not math.isfinite(norm_val):
            return False, norm_val, None
        clip = 1.0
        if cfg.clip_grad and cfg.clip_grad > 0:
            clip = min(1.0, cfg.clip_grad / (norm_val + 1e-6))
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        wd = self.param_groups[0]["weight_decay"]
        if cfg.cpu_offload:
            self._offload_fetch_grads()
        for sh in self.shards:
            g = sh.buf.grad_data[sh.start:sh.end]
            out = sh.buf.param_data[sh.start:sh.end]
            out_arg = out if out.dtype == torch.bfloat16 else None
            if sh.offload:
                self._offload_update(sh, out, lr, wd, clip)
                continue
            # runs of equal weight-decay setting -> one fused launch each
            runs = []
            for lo, hi, use_wd, *_ in sh.segments:
                if runs and runs[-1][2] == use_wd and runs[-1][1] >= lo - 64:
                    runs[-1][1] = hi
                else:
                    runs.append([lo, hi, use_wd])
            for lo, hi, use_wd in runs:
                if cfg.optimizer == "sgd":
                    # v = mu v + (g + wd w); w -= lr v   (momentum kept in the first-moment buffer)
                    w, v = sh.master[lo:hi], sh.exp_avg[lo:hi]
                    d = g[lo:hi].float() * clip
                    if use_wd and wd:
                        d = d + wd * w
                    v.copy_((cfg.sgd_momentum * v.float() + d).to(v.dtype))
                    w.add_(v.float(), alpha=-lr)
                    out[lo:hi].copy_(w)
                    continue
                if self._peer_ok(sh):
                    self._peer_adam_and_gather(sh, lo, hi, lr, wd if use_wd else 0.0, clip)
                    continue
                if sh.remainder:
                    OF.adam_step_remainder(out[lo:hi], sh.lo[lo:hi], g[lo:hi], sh.exp_avg[lo:hi],
                                           sh.exp_avg_sq[lo:hi], lr=lr, beta1=cfg.adam_beta1, beta2=cfg.adam_beta2,
                                           eps=cfg.adam_eps, weight_decay=wd if use_wd else 0.0,
                                           step=self.step_count, grad_scale=clip)
                    continue
                OF.adam_step(sh.master[lo:hi], g[lo:hi], sh.exp_avg[lo:hi], sh.exp_avg_sq[lo:hi],
                             out_arg[lo:hi] if out_arg is not None else None, lr=lr, beta1=cfg.adam_beta1,
                             beta2=cfg.adam_beta2, eps=cfg.adam_eps, weight_decay=wd if use_wd else 0.0,
                             step=self.step_count, grad_scale=clip)
                if out_arg is None:
                    out[lo:hi].copy_(sh.master[lo:hi])
        if cfg.cpu_offload and self._offload_stream is not None:
            torch.cuda.current_stream().wait_stream(self._offload_stream)
        self._gather_params()
        done = set()
        for sh in self._peer_buffers():  # pushes landed everywhere; gradients may be zeroed for the next step
            if id(sh.buf) not in done:
                self._peer_barrier(sh.buf)
                done.add(id(sh.buf))
        return True, norm_val, None

    # ------------------------------------------------------------------ host (offloaded) update
    def _offload_fetch_grads(self) -> None:
        """Queue every shard's gradient copy to pinned host memory on a side stream; each shard's host update then
        waits only for its own copy, so later copies overlap earlier updates."""
        dev = self.shards[0].buf.grad_data
        if dev.is_cuda and self._offload_stream is None:
            self._offload_stream = torch.cuda.Stream()
        for sh in self.shards:
            if not sh.offload:
                continue
            g = sh.buf.grad_data[sh.start:sh.end]
            if g.is_cuda:
                self._offload_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._offload_stream):
                    sh.host_grad.copy_(g.to(sh.host_grad.dtype), non_blocking=True)
                    sh.grad_event = torch.cuda.Event()
                    sh.grad_event.record(self._offload_stream)
            else:
                sh.host_grad.copy_(g)

    def _offload_update(self, sh, out, lr, wd, clip) -> None:
        from ..optim.cpu_offload import _load_ext

        ext, cfg = _load_ext(), self.cfg
        if sh.grad_event is not None:
            sh.grad_event.synchronize()
        runs = []
        for lo, hi, use_wd, *_ in sh.segments:
            if runs and runs[-1][2] == use_wd and runs[-1][1] == lo:
                runs[-1][1] = hi
            else:
                runs.append([lo, hi, use_wd])
        for lo, hi, use_wd in runs:
            ext.cpu_adam_step(sh._master[lo:hi], sh.host_grad[lo:hi], sh.exp_avg[lo:hi], sh.exp_avg_sq[lo:hi],
                              sh.host_out[lo:hi] if sh.host_out is not None else None, lr, cfg.adam_beta1,
                              cfg.adam_beta2, cfg.adam_eps, wd if use_wd else 0.0, self.step_count, clip)
            src = sh.host_out if sh.host_out is not None else sh._master
            if out.is_cuda:
                with torch.cuda.stream(self._offload_stream):
                    out[lo:hi].copy_(src[lo:hi], non_blocking=True)
            else:
                out[lo:hi].copy_(src[lo:hi])

    def _gather_params(self):
        """Refresh every rank's copy of the parameters from the owners' shards. With ``overlap_param_gather`` on a GPU
        the bucket all-gathers are only QUEUED here, on a communication stream and in the order the next forward pass
        needs them (the buffers hold the parameters in roughly backward order, so the last bucket goes first); each
        module waits for the buckets of its own parameters right before its forward (``_install_gather_waits``), so
        the transfer of the later layers hides under the compute of the earlier ones
        (reference: loongforge/train/training_utils.py:943-991,1319-1339)."""
        if not self.sharded:
            return
        todo = [sh for sh in self.shards if sh.buf.dp_size > 1 and not self._peer_ok(sh)]
        overlap = self.cfg.overlap_param_gather and todo and todo[0].buf.param_data.is_cuda
        if overlap:
            self._install_gather_waits()
            if self._gather_stream is None:
                self._gather_stream = torch.cuda.Stream()
            cur = torch.cuda.current_stream()
            self._gather_stream.wait_stream(cur)  # the updated shards are written by kernels of this stream
            with torch.cuda.stream(self._gather_stream):
                for sh in reversed(todo):
                    buf, b = sh.buf, sh.bucket
                    dist.all_gather_into_tensor(buf.param_data[b.start:b.end], buf.param_data[sh.start:sh.end],
                                                group=buf.dp_group)
                    ev = torch.cuda.Event()
                    ev.record(self._gather_stream)
                    self._gather_events[(id(buf), b.index)] = ev
            return
        for sh in todo:
            buf, b = sh.buf, sh.bucket
            full = buf.param_data[b.start:b.end]
            mine = buf.param_data[sh.start:sh.end]
            if full.is_cuda:
                dist.all_gather_into_tensor(full, mine, group=buf.dp_group)
            else:
                parts = list(full.chunk(buf.dp_size))
                dist.all_gather(parts, mine.clone(), group=buf.dp_group)

    def wait_param_gather(self, params=None) -> None:
        """Make the current stream wait for the queued all-gathers of the buckets that hold `params` (all pending
        buckets when None): called by the forward pre-hooks, and by anything that reads parameters outside a forward
        pass (checkpoint save, evaluation of parameter norms, weight hashing)."""
        if not self._gather_events:
            return
        if params is None:
            keys = list(self._gather_events)
        else:
            keys = {self._param_bucket.get(id(p)) for p in params}
        cur = torch.cuda.current_stream()
        for k in keys:
            ev = self._gather_events.pop(k, None) if k is not None else None
            if ev is not None:
                cur.wait_event(ev)

    def _install_gather_waits(self) -> None:
        if self._gather_hooks_installed:
            return
        self._gather_hooks_installed = True
        for m in self.models:
            for buf in m._all_buffers:
                for p, (_, _, bi) in buf.param_index.items():
                    self._param_bucket[id(p)] = (id(buf), bi)
            # Granularity: the members of every nn.ModuleList (transformer layers, experts) wait for the parameters of
            # their whole subtree right before they run; everything else (embedding, final norm, output layer, heads
            # whose weights the model reads without calling the sub-module) is awaited when the model's forward starts.
            layered = set()
            for mod in m.module.modules():
                if isinstance(mod, torch.nn.ModuleList):
                    for child in mod:
                        sub = list(child.parameters())
                        if sub:
                            layered.update(id(p) for p in sub)
                            child.register_forward_pre_hook(
                                lambda _m, _a, _sub=sub: self.wait_param_gather(_sub))
            rest = [p for p in m.module.parameters() if id(p) not in layered]
            m.module.register_forward_pre_hook(lambda _m, _a, _rest=rest: self.wait_param_gather(_rest))

    def zero_grad(self):
        for m in self.models:
            m.zero_grad_buffer()

    def reload_model_params(self):
        """Refresh fp32 masters from the (possibly just loaded) model weights."""
        for sh in self.shards:
            if sh.remainder:
                sh.lo.zero_()
            else:
                sh._master.copy_(sh.buf.param_data[sh.start:sh.end].float())

    # ------------------------------------------------------------------ checkpoint state
    def sharded_state(self) -> Dict[str, Dict[str, torch.Tensor]]:
        """Per-parameter optimizer-state pieces owned by this rank.

        Returns {param_name: [{"offset": int (into the flattened local param), "param", "master", "exp_avg",
        "exp_avg_sq"}]} which the checkpoint layer writes as flat shards with global offsets
        ("fully reshardable": a different DP size can re-assemble them). With several model chunks (virtual
        pipeline stages) the chunk-local names repeat, so they are prefixed ``chunk{i}.``; ``param`` identifies
        the tensor unambiguously."""
        out = {}
        many = len(self.models) > 1
        for sh in self.shards:
            for lo, hi, _, _, name, p, pstart in sh.segments:
                off = sh.start + lo - pstart
                out.setdefault(f"chunk{sh.chunk}.{name}" if many else name, []).append({
                    "offset": off, "numel": hi - lo, "param_numel": p.numel(), "param": p,
                    "master": sh.master[lo:hi], "exp_avg": sh.exp_avg[lo:hi], "exp_avg_sq": sh.exp_avg_sq[lo:hi],
                    "set_master": (lambda v, sh=sh, lo=lo, hi=hi: sh.set_master(lo, hi, v))})
        return out

    def state_dict(self):
        return {"step": self.step_count, "param_groups": self.param_groups}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.param_groups = sd["param_groups"]

    def load_sharded_state(self, pieces_by_name):
        """Inverse of :meth:`sharded_state`; `pieces_by_name[name]` is a dict of full flat tensors
        (local parameter numel) for master / exp_avg / exp_avg_sq."""
        many = len(self.models) > 1
        for sh in self.shards:
            for lo, hi, _, _, name, p, pstart in sh.segments:
                src = pieces_by_name.get(f"chunk{sh.chunk}.{name}" if many else name)
                if src is None:
                    continue
                off = sh.start + lo - pstart
                sh.set_master(lo, hi, src["master"][off:off + hi - lo])
                sh.exp_avg[lo:hi].copy_(src["exp_avg"][off:off + hi - lo])
                sh.exp_avg_sq[lo:hi].copy_(src["exp_avg_sq"][off:off + hi - lo])
