"""Sequence-parallel linears fused with their collective over NVLink peer memory.

``all_gather_linear``  : Y = all_gather(X) @ W^T       (QKV / FC1 column-parallel linears)
``linear_reduce_scatter``: Y = reduce_scatter(X @ W^T) (+ residual)  (proj / FC2 row-parallel)

Each direction is ONE kernel launch per rank (``csrc/peer_gemm.cu``); the backward passes use the
same two kernels with the weight read MN-major:

    all_gather_linear.backward    : dX = reduce_scatter(dY @ W)      -> gemm_rs
                                    dW = dY^T @ all_gather(X)        -> plain GEMM on the saved gather
    linear_reduce_scatter.backward: dX = all_gather(dY) @ W          -> ag_gemm
                                    dW = all_gather(dY)^T @ X        -> plain GEMM on that gather

Peer buffers are symmetric allocations (same layout on every rank) obtained once per
(shape, group) through ``torch.distributed._symmetric_memory`` and reused by every layer; they are
double buffered by call parity so that no cross-rank barrier is needed between calls. The NCCL
mappings in ``parallel/mappings.py`` remain the reference path (and the CPU path).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops import functional as OF
from . import state as ps

_COPY_CTAS = 8
_MAX_PEERS = 8


class _SymmetricBlock:
    """One symmetric allocation per rank, carved into named byte ranges; gives peer pointers."""

    def __init__(self, nbytes: int, group, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.nbytes = (nbytes + 255) // 256 * 256
        self.tensor = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def peer_ptrs(self, offset: int):
        return [p + offset for p in self.ptrs]

    def local_view(self, offset: int, nbytes: int, dtype, shape):
        return self.tensor[offset:offset + nbytes].view(dtype).view(shape)


class _AgContext:
    """Buffers of the all-gather->GEMM kernel for one (rows_per_rank, K) shape."""

    def __init__(self, rows: int, K: int, group, device):
        world = dist.get_world_size(group)
        full = rows * world * K * 2
        self.sync_off = 2 * full
        # two (call parity) symmetric [T, K] gather buffers: every rank writes its own rows in place and pulls the
        # peers' rows from the same offsets of their buffers
        self.block = _SymmetricBlock(2 * full + 256, group, device)
        self.rows, self.K = rows, K
        self.world, self.rank = self.block.world, self.block.rank
        self.full_bytes = full
        self.x_sym = [self.block.local_view(i * full, full, torch.bfloat16, (rows * world, K)) for i in range(2)]
        self.chunk_flags = torch.zeros(rows * self.world // 128, dtype=torch.int32, device=device)
        self.epoch = 0

    def next(self):
        self.epoch += 1
        par = self.epoch & 1
        return self.epoch, self.x_sym[par], self.block.peer_ptrs(par * self.full_bytes), \
            self.block.peer_ptrs(self.sync_off)


class _RsContext:
    """Receive buffers and tile counters of the GEMM->reduce-scatter kernel for one (T, N) shape."""

    def __init__(self, T: int, N: int, group, device, world: int):
        rows = T // world
        tiles = (rows // 128) * ((N + 255) // 256)
        recv = 2 * world * rows * N * 2
        flags = 2 * world * tiles * 4
        self.flags_off = (recv + 255) // 256 * 256
        self.block = _SymmetricBlock(self.flags_off + flags, group, device)
        self.world, self.rank = self.block.world, self.block.rank
        self.calls = 0

    def next(self):
        c = self.calls
        self.calls += 1
        return c, self.block.peer_ptrs(0), self.block.peer_ptrs(self.flags_off)


_ag_ctx: Dict[Tuple, _AgContext] = {}
_rs_ctx: Dict[Tuple, _RsContext] = {}


def _group(state_name):
    st = ps.get_state(state_name)
    return st, st.group("tp")


def _get_ag(rows, K, state_name, device) -> _AgContext:
    st, g = _group(state_name)
    key = (rows, K, st.name, device.index)
    if key not in _ag_ctx:
        _ag_ctx[key] = _AgContext(rows, K, g, device)
    return _ag_ctx[key]


def _get_rs(T, N, state_name, device) -> _RsContext:
    st, g = _group(state_name)
    key = (T, N, st.name, device.index)
    if key not in _rs_ctx:
        _rs_ctx[key] = _RsContext(T, N, g, device, st.dims.tp)
    return _rs_ctx[key]


def supported(x: torch.Tensor, weight: torch.Tensor, rows_per_rank: int) -> bool:
    m = _ext.get()
    return (m is not None and hasattr(m, "ag_gemm") and x.is_cuda and x.dtype == torch.bfloat16
            and rows_per_rank % 128 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0)


def _ag_gemm(x_shard: torch.Tensor, B: torch.Tensor, b_mn: bool, bias, state_name):
    """Returns (all_gather(x_shard) @ op(B), gathered x). The gathered tensor is a view of the symmetric gather buffer:
    it stays valid until the second-next call for the same shape, so consumers use it right away (same stream)."""
    rows, K = x_shard.shape
    ctx = _get_ag(rows, K, state_name, x_shard.device)
    epoch, x_full, peer_x, peer_sync = ctx.next()
    x_full[ctx.rank * rows:(ctx.rank + 1) * rows].copy_(x_shard)
    y = _ext.require().ag_gemm(peer_x, peer_sync, x_full, ctx.chunk_flags, B, b_mn, bias, ctx.rank, rows, epoch,
                               _COPY_CTAS, _ext.status_tensor(x_shard.device))
    return y, x_full


def _gemm_rs(a: torch.Tensor, B: torch.Tensor, b_mn: bool, residual, state_name):
    T = a.shape[0]
    N = B.shape[1] if b_mn else B.shape[0]
    ctx = _get_rs(T, N, state_name, a.device)
    call, peer_recv, peer_flags = ctx.next()
    return _ext.require().gemm_rs(a, B, b_mn, peer_recv, peer_flags, residual, ctx.rank, call,
                                  _ext.status_tensor(a.device))


_side_stream: Dict[int, torch.cuda.Stream] = {}


def _side(device) -> torch.cuda.Stream:
    s = _side_stream.get(device.index)
    if s is None:
        s = _side_stream[device.index] = torch.cuda.Stream(device=device)
    return s


class _AllGatherLinearFn(torch.autograd.Function):
    """Forward keeps only this rank's sequence shard (as Megatron's sequence parallelism does); backward gathers it
    again on a side stream while the input-gradient GEMM -> reduce-scatter kernel runs."""

    @staticmethod
    def forward(ctx, x, weight, bias, state_name):
        y, _ = _ag_gemm(x, weight, False, bias, state_name)
        ctx.save_for_backward(x, weight)
        ctx.state_name = state_name
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = db = None
        x_full = None
        if ctx.needs_input_grad[1]:
            _, g = _group(ctx.state_name)
            cur, side = torch.cuda.current_stream(), _side(x.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                x_full = torch.empty(x.shape[0] * dist.get_world_size(g), x.shape[1], dtype=x.dtype, device=x.device)
                dist.all_gather_into_tensor(x_full, x.contiguous(), group=g)
            x_full.record_stream(cur)
        if ctx.needs_input_grad[0]:
            dx = _gemm_rs(dy, weight, True, None, ctx.state_name)
        if ctx.needs_input_grad[1]:
            torch.cuda.current_stream().wait_stream(_side(x.device))
            dw = OF._wgrad(dy, x_full, weight)
        if ctx.has_bias:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


class _LinearReduceScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, state_name):
        y = _gemm_rs(x, weight, False, residual, state_name)
        ctx.save_for_backward(x, weight)
        ctx.state_name = state_name
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx, dy_full = _ag_gemm(dy, weight, True, None, ctx.state_name)
        dw = OF._wgrad(dy_full, x, weight) if ctx.needs_input_grad[1] else None
        return dx, dw, (dy if ctx.has_res else None), None


def all_gather_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state_name=None):
    """x ``[T/tp, in]`` (this rank's sequence shard) -> ``[T, out/tp]``."""
    if not supported(x, weight, x.shape[0]):
        from . import mappings as M
        _, g = _group(state_name)
        return OF.linear(M.gather_from_sequence_parallel_region(x, g, True), weight, bias)
    return _AllGatherLinearFn.apply(x.contiguous(), weight, bias, state_name)


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor], state_name=None):
    """x ``[T, in/tp]`` -> ``[T/tp, out]`` (+ residual of that shape)."""
    st, g = _group(state_name)
    if not supported(x, weight, x.shape[0] // st.dims.tp):
        from . import mappings as M
        y = M.reduce_scatter_to_sequence_parallel_region(OF.linear(x, weight), g)
        return y + residual if residual is not None else y
    return _LinearReduceScatterFn.apply(x.contiguous(), weight, residual, state_name)


def reset():
    _ag_ctx.clear()
    _rs_ctx.clear()
