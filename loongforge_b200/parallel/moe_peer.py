"""Expert-parallel token dispatcher over NVLink peer memory.

Replaces the NCCL all_to_all(v) + permute / unpermute pair of Megatron's alltoall dispatcher (used
by every MoE model of the reference through ``MoELayer``) with two kernels over symmetric memory
(``csrc/moe_peer.cu``):

* ``push``: every (token, expert) pair's hidden row is stored directly into its final expert-sorted
  row on the rank that owns the expert — dispatch, permutation and the sort by local expert in one
  pass — together with the pair's router probability;
* ``pull``: every token sums the rows of its k pairs, loaded from the owning ranks — combine,
  un-permute and top-k reduction in one pass with a fixed summation order.

The probability is applied on the expert side (after the activation, before FC2), so ``pull`` is an
unweighted sum and the backward of ``push`` is ``pull`` and vice versa; the router-probability
gradient comes back as one scalar per pair.

Protocol per call (all ranks execute the same sequence, forward and backward alike)::

    push(buffer A) -> flag A -> wait A -> experts -> copy into buffer B -> flag B -> wait B -> pull(B)

A rank may overwrite a peer's A only after that peer consumed it: the peer's flag B is released
after its experts ran, and the pusher waits for flag B before its next push. A rank overwrites its
own B only after waiting for every peer's next flag A, which peers release after their pull.

Row offsets come from the [ep, E] matrix of per-rank expert counts (one small all-gather) and one
host read of this rank's per-expert totals, which the grouped GEMM's tile table needs anyway.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _ext

KIND_A, KIND_B = 0, 1


class _LocalBlock:
    """Single-rank stand-in for the symmetric allocation (expert parallel size 1)."""

    def __init__(self, nbytes: int, device):
        self.tensor = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.rank, self.world = 0, 1

    def peer_ptrs(self, offset: int):
        return [self.tensor.data_ptr() + offset]

    def local_view(self, offset: int, nbytes: int, dtype, shape):
        return self.tensor[offset:offset + nbytes].view(dtype).view(shape)


class PeerExchange:
    """Symmetric buffers of one EP group: A and B row buffers [cap, H] bf16, scalars [cap] f32, flags."""

    _cache: Dict[Tuple, "PeerExchange"] = {}

    def __init__(self, group, device, hidden: int, cap_rows: int):
        from .fused_tp import _SymmetricBlock

        self.group, self.H, self.cap = group, hidden, cap_rows
        row_bytes = cap_rows * hidden * 2
        scal_bytes = (cap_rows * 4 + 255) // 256 * 256
        self.off_a, self.off_b = 0, row_bytes
        self.off_sa, self.off_sb = 2 * row_bytes, 2 * row_bytes + scal_bytes
        self.off_flags = 2 * row_bytes + 2 * scal_bytes
        if group is None:
            self.block = _LocalBlock(self.off_flags + 256, device)
        else:
            self.block = _SymmetricBlock(self.off_flags + 256, group, device)
        self.rank, self.world = self.block.rank, self.block.world
        self.buf_a = self.block.local_view(self.off_a, row_bytes, torch.bfloat16, (cap_rows, hidden))
        self.buf_b = self.block.local_view(self.off_b, row_bytes, torch.bfloat16, (cap_rows, hidden))
        self.scal_a = self.block.local_view(self.off_sa, cap_rows * 4, torch.float32, (cap_rows,))
        self.scal_b = self.block.local_view(self.off_sb, cap_rows * 4, torch.float32, (cap_rows,))
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = {KIND_A: 0, KIND_B: 0}
        self.flags = self.block.peer_ptrs(self.off_flags)

    @classmethod
    def get(cls, group, device, hidden: int, cap_rows: int, headroom: float = 1.0) -> "PeerExchange":
        """The group's exchange if it holds `cap_rows` rows, else a new one of ``cap_rows * headroom`` rows. Allocation
        is collective: every rank of the group must reach this call with the SAME `cap_rows` and `headroom`."""
        key = (id(group), str(device), hidden)
        ex = cls._cache.get(key)
        if ex is None or ex.cap < cap_rows:
            ex = cls(group, device, hidden, int(cap_rows * max(headroom, 1.0)) + 128)
            cls._cache[key] = ex
        return ex

    def ptrs(self, which: str):
        if which == "a":
            return self.block.peer_ptrs(self.off_a), self.block.peer_ptrs(self.off_sa)
        return self.block.peer_ptrs(self.off_b), self.block.peer_ptrs(self.off_sb)

    def bump(self, kind: int) -> int:
        self.epoch[kind] += 1
        return self.epoch[kind]


class RoutePlan:
    """Device-side index arrays of one routing decision (no host sync except `tokens_per_expert`)."""

    def __init__(self, topk_idx: torch.Tensor, num_experts: int, ep: int, ep_rank: int, group, cap_rows: int,
                 all_counts: Optional[torch.Tensor] = None):
        """``all_counts`` [ep, E] (tokens of every rank per global expert) is gathered over ``group`` when not given."""
        T, k = topk_idx.shape
        dev = topk_idx.device
        E, El = num_experts, num_experts // ep
        flat = topk_idx.reshape(-1).long()
        sorted_e, perm = torch.sort(flat, stable=True)          # pair j <-> slot perm[j] = t * k + kk
        counts = torch.bincount(flat, minlength=E)              # my tokens per global expert
        start = torch.cumsum(counts, 0) - counts
        if all_counts is not None:
            pass
        elif ep > 1:
            all_counts = torch.empty(ep, E, dtype=counts.dtype, device=dev)
            dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=group)
        else:
            all_counts = counts.view(1, E)
        # blocks[d, e_local, s] = rows rank s sends to local expert e_local of rank d; rows at d are laid out
        # in (e_local, s) order
        blocks = all_counts.view(ep, ep, El).permute(1, 2, 0).contiguous()
        flat_blocks = blocks.view(ep, El * ep)
        offs = (torch.cumsum(flat_blocks, 1) - flat_blocks).view(ep, El, ep)
        base = offs[:, :, ep_rank].reshape(E)                   # first row of my block for global expert e
        host = torch.cat([blocks[ep_rank].sum(-1), flat_blocks.sum(1).max().view(1)]).tolist()  # one D2H
        self.tokens_per_expert: List[int] = [int(v) for v in host[:El]]
        self.rows = sum(self.tokens_per_expert)
        # most rows any rank of the group receives; identical on every rank, so all ranks grow their buffers together
        self.max_rows = int(host[-1])
        j = torch.arange(T * k, device=dev)
        self.pair_token = (perm // k).int()
        self.pair_row = (base[sorted_e] + (j - start[sorted_e])).int()
        self.pair_dst = (sorted_e // El).int()
        self.slot_pair = torch.empty(T * k, dtype=torch.int32, device=dev)
        self.slot_pair[perm] = j.int()
        self.pair_expert = sorted_e
        self.T, self.k = T, k


class _Dispatch(torch.autograd.Function):
    """x [T, H], pair_probs [P] -> (tokens [R, H] sorted by local expert, row_probs [R])."""

    @staticmethod
    def forward(ctx, x, pair_probs, ex: PeerExchange, plan: RoutePlan):
        C = _ext.require()
        st = _ext.status_tensor(x.device)
        bufs, scal = ex.ptrs("a")
        ep_a = ex.bump(KIND_A)
        C.moe_push(bufs, scal, ex.flags, ex.rank, ex.cap, x.contiguous(), plan.pair_token, plan.pair_row, plan.pair_dst,
                   pair_probs.float().contiguous(), ex.done, KIND_A, ep_a, st)
        C.moe_wait(bufs, scal, ex.flags, ex.rank, KIND_A, ep_a, st)
        tokens = ex.buf_a[:plan.rows].clone()
        row_probs = ex.scal_a[:plan.rows].clone()
        ctx.ex, ctx.plan = ex, plan
        return tokens, row_probs

    @staticmethod
    def backward(ctx, d_tokens, d_row_probs):
        ex, plan = ctx.ex, ctx.plan
        C = _ext.require()
        st = _ext.status_tensor(d_tokens.device)
        bufs, scal = ex.ptrs("b")
        ex.buf_b[:plan.rows].copy_(d_tokens)
        ex.scal_b[:plan.rows].copy_(d_row_probs)
        ep_b = ex.bump(KIND_B)
        C.moe_signal(bufs, scal, ex.flags, ex.rank, KIND_B, ep_b)
        C.moe_wait(bufs, scal, ex.flags, ex.rank, KIND_B, ep_b, st)
        dx, dslot = C.moe_pull(bufs, scal, ex.flags, ex.rank, ex.cap, plan.T, plan.k, ex.H, plan.slot_pair,
                               plan.pair_row, plan.pair_dst, True, st)
        d_pair = torch.empty_like(dslot.view(-1))
        d_pair[plan.slot_pair.long()] = dslot.view(-1)
        return dx, d_pair, None, None


class _Combine(torch.autograd.Function):
    """y [R, H] (expert outputs, already probability weighted) -> out [T, H] = sum over each token's pairs."""

    @staticmethod
    def forward(ctx, y, ex: PeerExchange, plan: RoutePlan):
        C = _ext.require()
        st = _ext.status_tensor(y.device)
        bufs, scal = ex.ptrs("b")
        ex.buf_b[:plan.rows].copy_(y)
        ep_b = ex.bump(KIND_B)
        C.moe_signal(bufs, scal, ex.flags, ex.rank, KIND_B, ep_b)
        C.moe_wait(bufs, scal, ex.flags, ex.rank, KIND_B, ep_b, st)
        out, _ = C.moe_pull(bufs, scal, ex.flags, ex.rank, ex.cap, plan.T, plan.k, ex.H, plan.slot_pair, plan.pair_row,
                            plan.pair_dst, False, st)
        ctx.ex, ctx.plan = ex, plan
        return out

    @staticmethod
    def backward(ctx, d_out):
        ex, plan = ctx.ex, ctx.plan
        C = _ext.require()
        st = _ext.status_tensor(d_out.device)
        bufs, scal = ex.ptrs("a")
        ep_a = ex.bump(KIND_A)
        C.moe_push(bufs, scal, ex.flags, ex.rank, ex.cap, d_out.contiguous(), plan.pair_token, plan.pair_row,
                   plan.pair_dst, None, ex.done, KIND_A, ep_a, st)
        C.moe_wait(bufs, scal, ex.flags, ex.rank, KIND_A, ep_a, st)
        return ex.buf_a[:plan.rows].clone(), None, None


class PeerDispatcher:
    """Drop-in for the all-to-all dispatcher on CUDA. ``dispatch`` returns the probabilities of the received
    rows as a third value: the expert MLP multiplies them in before FC2."""

    weights_on_expert_side = True

    def __init__(self, num_experts: int, hidden: int, ep: int, ep_rank: int, group, capacity_factor: float = 2.0):
        self.E, self.H, self.ep, self.ep_rank, self.group = num_experts, hidden, ep, ep_rank, group
        self.capacity_factor = capacity_factor
        self.ex: Optional[PeerExchange] = None
        self.plan: Optional[RoutePlan] = None

    def dispatch(self, x: torch.Tensor, probs: torch.Tensor, topk_idx: torch.Tensor):
        self.plan = RoutePlan(topk_idx, self.E, self.ep, self.ep_rank, self.group, 0)
        # The buffers are sized from the most rows ANY rank receives: that number comes from the all-gathered counts
        # and is the same on every rank, whatever each rank's own token count, so all ranks (re-)allocate the symmetric
        # buffers at the same call. The capacity factor is the headroom kept above it when allocating.
        self.ex = PeerExchange.get(self.group, x.device, self.H, max(self.plan.max_rows, 128),
                                   headroom=max(self.capacity_factor, 1.25))
        pair_probs = probs[self.plan.pair_token.long(), self.plan.pair_expert]
        tokens, row_probs = _Dispatch.apply(x, pair_probs, self.ex, self.plan)
        return tokens, self.plan.tokens_per_expert, row_probs

    def combine(self, y: torch.Tensor) -> torch.Tensor:
        return _Combine.apply(y, self.ex, self.plan)
