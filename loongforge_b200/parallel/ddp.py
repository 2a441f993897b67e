"""Data-parallel wrapper with contiguous parameter / gradient buffers and bucketed,
overlapped gradient reduction.

Re-creates Megatron's ``DistributedDataParallel`` semantics that the reference configures in
loongforge/train/training_utils.py:943-991: parameters of one dtype live in one flat buffer,
gradients accumulate in a flat ``main_grad`` buffer (fp32 by default), the buffer is cut into
buckets of at least ``bucket_size`` elements in reverse parameter order, and a bucket's
reduce-scatter (distributed optimizer) or all-reduce starts as soon as every gradient in it is
ready on the last micro-batch (``overlap_grad_reduce``). Expert parameters use the
expert-data-parallel group in their own buffer.
"""
from __future__ import annotations

import contextlib
import dataclasses
import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import state as ps


@dataclasses.dataclass
class DDPConfig:
    grad_reduce_in_fp32: bool = True
    overlap_grad_reduce: bool = True
    use_distributed_optimizer: bool = True
    bucket_size: Optional[int] = 40_000_000
    average_in_collective: bool = False
    check_for_nan_in_grad: bool = False
    align_elems: int = 128
    # parameter / gradient buffers in symmetric (peer-mappable) memory and NO NCCL gradient reduce-scatter: the
    # distributed optimizer then reduces by peer loads and all-gathers by peer stores inside its own kernels
    peer_optimizer: bool = False


@dataclasses.dataclass
class Bucket:
    index: int
    start: int  # element offsets into the flat buffer
    end: int
    params: List[nn.Parameter]
    pending: set
    handle: Optional[object] = None
    shard_out: Optional[torch.Tensor] = None


class ParamAndGradBuffer:
    """Flat storage for a set of parameters that share dtype and data-parallel group."""

    def __init__(self, params: List[nn.Parameter], named: Dict[nn.Parameter, str], cfg: DDPConfig, dp_group,
                 dp_size: int, dp_rank: int, param_dtype: torch.dtype, grad_dtype: torch.dtype,
                 grad_scale: Optional[float] = None):
        self.cfg, self.dp_group, self.dp_size, self.dp_rank = cfg, dp_group, dp_size, dp_rank
        # Gradients are AVERAGED over the full data-parallel size. Expert parameters are reduced over
        # the (smaller) expert-data-parallel group but already hold the token contributions of all
        # expert-parallel ranks, so they are scaled by 1/dp as well, not 1/edp.
        self.grad_scale = (1.0 / dp_size) if grad_scale is None else grad_scale
        self.param_dtype, self.grad_dtype = param_dtype, grad_dtype
        self.params = list(reversed(params))  # roughly backward order
        self.named = named
        device = self.params[0].device
        # bucket boundaries: close a bucket once it holds >= bucket_size elements
        align = cfg.align_elems * (dp_size if cfg.use_distributed_optimizer else 1)
        align = math.lcm(align, dp_size)
        self.param_index: Dict[nn.Parameter, tuple] = {}
        self.buckets: List[Bucket] = []
        off = 0
        b_start, b_params = 0, []

        def close():
            nonlocal off, b_start, b_params
            if not b_params:
                return
            off = ((off + align - 1) // align) * align
            self.buckets.append(Bucket(len(self.buckets), b_start, off, b_params, set()))
            b_start, b_params = off, []

        for p in self.params:
            n = p.numel()
            start = off
            off += n
            # keep every parameter 16-byte aligned for TMA / vector access
            off = ((off + 63) // 64) * 64
            self.param_index[p] = (start, start + n, len(self.buckets))
            b_params.append(p)
            if cfg.bucket_size is not None and (off - b_start) >= cfg.bucket_size:
                close()
        close()
        self.numel = off
        self.symmetric = None
        if cfg.peer_optimizer and dp_size > 1 and torch.device(device).type == "cuda":
            # one symmetric allocation: [params | grads | 2 x int[8] arrival flags]
            from .fused_tp import _SymmetricBlock
            pb = (self.numel * torch.empty(0, dtype=param_dtype).element_size() + 255) // 256 * 256
            gb = (self.numel * torch.empty(0, dtype=grad_dtype).element_size() + 255) // 256 * 256
            blk = _SymmetricBlock(pb + gb + 256, dp_group, device)
            self.symmetric = {"block": blk, "param_off": 0, "grad_off": pb, "flag_off": pb + gb, "epoch": 0}
            self.param_data = blk.local_view(0, self.numel * torch.empty(0, dtype=param_dtype).element_size(),
                                             param_dtype, (self.numel,))
            self.grad_data = blk.local_view(pb, self.numel * torch.empty(0, dtype=grad_dtype).element_size(),
                                            grad_dtype, (self.numel,))
        else:
            self.param_data = torch.zeros(self.numel, dtype=param_dtype, device=device)
            self.grad_data = torch.zeros(self.numel, dtype=grad_dtype, device=device)
        for p in self.params:
            s, e, _ = self.param_index[p]
            self.param_data[s:e].view(p.shape).copy_(p.data)
            p.data = self.param_data[s:e].view(p.shape)
            p.main_grad = self.grad_data[s:e].view(p.shape)
            p.grad_added_to_main_grad = False

    def shard_range(self, bucket: Bucket) -> tuple:
        n = (bucket.end - bucket.start) // self.dp_size
        s = bucket.start + self.dp_rank * n
        return s, s + n


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, cfg: Optional[DDPConfig] = None, parallel_state: Optional[str] = None,
                 disable_bucketing: bool = False):
        super().__init__()
        self.module = module
        self.cfg = cfg or DDPConfig()
        st = ps.get_state(parallel_state)
        self.state = st
        if disable_bucketing:
            self.cfg = dataclasses.replace(self.cfg, bucket_size=None)
        dense, expert, shared, mp_shared = [], [], [], []
        named = {}
        for name, p in module.named_parameters():
            if not p.requires_grad:
                continue
            named[p] = name
            if getattr(p, "shared_embedding", False):
                shared.append(p)
            elif getattr(p, "mp_shared", False):
                mp_shared.append(p)  # replicated over the whole model-parallel group (vision encoder, full hetero-DP)
            else:
                (expert if getattr(p, "is_expert", False) else dense).append(p)
        self.buffers: List[ParamAndGradBuffer] = []
        self.expert_buffers: List[ParamAndGradBuffer] = []
        # The word embedding that the first and last pipeline stage both hold lives in a buffer of its own: both
        # stages then shard it identically over the data-parallel ranks, so its gradient can be summed over the two
        # stages after the data-parallel reduce-scatter (reference: Megatron gives such parameters their own bucket).
        for plist, kind, store in ((dense, "dp_cp", self.buffers), (shared, "dp_cp", self.buffers),
                                   (mp_shared, "dp_cp", self.buffers), (expert, "edp", self.expert_buffers)):
            by_dtype: Dict[torch.dtype, List[nn.Parameter]] = {}
            for p in plist:
                by_dtype.setdefault(p.dtype, []).append(p)
            for dt, ps_ in by_dtype.items():
                gdt = torch.float32 if self.cfg.grad_reduce_in_fp32 else dt
                store.append(ParamAndGradBuffer(ps_, named, self.cfg, st.group(kind), st.size(kind),
                                                st.rank_in(kind), dt, gdt, grad_scale=1.0 / st.size("dp_cp")))
        self._all_buffers = self.buffers + self.expert_buffers
        self.is_last_microbatch = True
        self._comm_stream = None
        self._hooks = []
        for buf in self._all_buffers:
            for p in buf.params:
                p.grad_ready = self._make_ready(buf, p)
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_accumulate_hook(buf, p)))
        self._reset_pending()

    # ------------------------------------------------------------------ hooks
    def _make_accumulate_hook(self, buf, p):
        def hook(param):
            # ops that accumulate straight into main_grad return no gradient, so whatever arrives here is a
            # contribution that is not in main_grad yet (e.g. the embedding lookup of a weight tied to the output layer)
            if param.grad is not None:
                param.main_grad.add_(param.grad.to(param.main_grad.dtype))
                param.grad = None
            param.grad_ready()
        return hook

    def _make_ready(self, buf: ParamAndGradBuffer, p):
        def ready():
            if not self.is_last_microbatch or not self.cfg.overlap_grad_reduce:
                return
            if getattr(p, "defer_grad_sync", False):
                return  # several gradient sources per backward: reduced when the backward pass has finished
            b = buf.buckets[buf.param_index[p][2]]
            b.pending.discard(p)
            if not b.pending and b.handle is None:
                self._start_bucket(buf, b)
        return ready

    def _reset_pending(self):
        for buf in self._all_buffers:
            for b in buf.buckets:
                b.pending = set(b.params)
                b.handle = None
                b.shard_out = None

    # ------------------------------------------------------------------ communication
    def _start_bucket(self, buf: ParamAndGradBuffer, b: Bucket, async_op: bool = True):
        g = buf.grad_data[b.start:b.end]
        scale = buf.grad_scale
        if buf.symmetric is not None:
            b.handle = True  # reduced (and scaled) by the optimizer's pull kernel at step time
            return
        if buf.dp_size == 1:
            if scale != 1.0:
                g.mul_(scale)
            b.handle = True
            return
        use_avg = self.cfg.average_in_collective and g.is_cuda and abs(scale * buf.dp_size - 1.0) < 1e-12
        if not use_avg:
            g.mul_(scale)
        op = dist.ReduceOp.AVG if use_avg else dist.ReduceOp.SUM
        if g.is_cuda and async_op:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream()
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                self._collective(buf, b, g, op)
            b.handle = self._comm_stream
        else:
            self._collective(buf, b, g, op)
            b.handle = True

    def _collective(self, buf, b, g, op):
        if self.cfg.use_distributed_optimizer:
            s, e = buf.shard_range(b)
            out = buf.grad_data[s:e]
            if g.is_cuda:
                dist.reduce_scatter_tensor(out, g, op=op, group=buf.dp_group)
            else:
                dist.all_reduce(g, op=op, group=buf.dp_group)
        else:
            dist.all_reduce(g, op=op, group=buf.dp_group)

    def start_grad_sync(self):
        for buf in self._all_buffers:
            for b in buf.buckets:
                if b.handle is None:
                    self._start_bucket(buf, b)

    def finish_grad_sync(self):
        """Make sure every bucket was reduced and the compute stream sees the results."""
        self.start_grad_sync()
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        self._reset_pending()

    # ------------------------------------------------------------------ API
    @contextlib.contextmanager
    def no_sync(self):
        prev = self.is_last_microbatch
        self.is_last_microbatch = False
        try:
            yield
        finally:
            self.is_last_microbatch = prev

    def zero_grad_buffer(self):
        for buf in self._all_buffers:
            buf.grad_data.zero_()
            for p in buf.params:
                p.grad_added_to_main_grad = False
        self._reset_pending()

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def state_dict(self, *a, **kw):
        return self.module.state_dict(*a, **kw)

    def load_state_dict(self, sd, strict: bool = True):
        return self.module.load_state_dict(sd, strict=strict)

    def broadcast_params(self):
        """Make the replicas identical at start-up (rank 0 of each DP group wins)."""
        for buf in self._all_buffers:
            if buf.dp_size > 1:
                src = dist.get_process_group_ranks(buf.dp_group)[0]
                dist.broadcast(buf.param_data, src=src, group=buf.dp_group)
