"""Context parallelism: load-balanced sequence sharding of the batch and three attention
communication schemes.

* ``get_batch_on_this_cp_rank`` / ``cp_chunk_indices``: each sequence is cut into ``2*cp`` chunks and
  rank r keeps chunks ``r`` and ``2*cp-1-r`` (causal load balance), the input preparation the
  reference does in loongforge/models/omni_models/utils.py:26-184 and
  loongforge/train/pretrain/pretrain_llm.py:70.
* ``cp_comm_type``:
    - ``"p2p"``      ring of KV blocks with online-softmax merging of partial results;
    - ``"allgather"`` K/V all-gathered once (backward reduce-scatters dK/dV);
    - ``"a2a+p2p"``   two levels: Ulysses inside blocks of neighbouring ranks, the ring between the blocks
    - ``"a2a"``       Ulysses: all-to-all from sequence-sharded/all-heads to full-sequence/head-sharded,
                      the ordinary attention kernel, and the inverse all-to-all
                      (loongforge/train/validators.py:391-433 maps --context-parallel-ulysses-degree here).
  On an NVSwitch node every peer is one hop away, so ``a2a`` keeps the tcgen05 attention kernel on
  full sequences and is the default when the head counts divide; the ring is kept for head counts
  that do not.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from . import mappings as M
from . import state as ps

_CFG = {"comm_type": "auto"}


def set_cp_comm_type(name: str, ulysses_degree: Optional[int] = None):
    """``"a2a+p2p"`` is the two-level scheme: Ulysses all-to-all among `ulysses_degree` neighbouring ranks, the KV
    ring between those blocks. Its process groups are created here, so every rank of the job must make this call."""
    assert name in ("auto", "p2p", "allgather", "a2a", "a2a+p2p")
    _CFG["comm_type"], _CFG["ulysses_degree"] = name, ulysses_degree
    if name == "a2a+p2p" and ps.model_parallel_is_initialized():
        ensure_cp_groups()


def ensure_cp_groups() -> None:
    """Create the process groups of the two-level scheme once the parallel state exists (the trainers call this right
    after they initialise it; a no-op for the other communication types)."""
    if _CFG["comm_type"] != "a2a+p2p":
        return
    st = ps.get_state()
    u = _CFG.get("ulysses_degree")
    if not u or st.dims.cp % u:
        raise ValueError("a2a+p2p needs a Ulysses degree that divides the context parallel size")
    if u == st.dims.cp:
        _CFG["comm_type"] = "a2a"
    elif u == 1:
        _CFG["comm_type"] = "p2p"
    elif "cp_inner" not in st.groups:
        st.create_hierarchical_cp_groups(u)


def cp_chunk_indices(seq_len: int, cp: int, rank: int, device=None) -> torch.Tensor:
    """Token indices (ascending) of the two chunks owned by `rank`."""
    assert seq_len % (2 * cp) == 0, "sequence length must divide by 2*cp"
    L = seq_len // (2 * cp)
    a = torch.arange(rank * L, (rank + 1) * L, device=device)
    b = torch.arange((2 * cp - 1 - rank) * L, (2 * cp - rank) * L, device=device)
    return torch.cat([a, b])


def get_batch_on_this_cp_rank(batch: Dict[str, torch.Tensor], cp: Optional[int] = None, rank: Optional[int] = None,
                              seq_dim: int = 1) -> Dict[str, torch.Tensor]:
    st = ps.get_state()
    cp = st.dims.cp if cp is None else cp
    rank = st.cp_rank if rank is None else rank
    if cp == 1:
        return batch
    out = {}
    for k, v in batch.items():
        if isinstance(v, torch.Tensor) and v.dim() > seq_dim and k in ("tokens", "labels", "loss_mask", "position_ids"):
            idx = cp_chunk_indices(v.shape[seq_dim], cp, rank, v.device)
            out[k] = v.index_select(seq_dim, idx)
        else:
            out[k] = v
    return out


def _masked_attention(q, k, v, q_pos, k_pos, scale, causal, seg_q=None, seg_k=None, return_lse=False):
    """Attention with an explicit position mask (fp32 softmax). q [Tq, Hq, D], k/v [Tk, Hkv, D]."""
    Hq, Hkv = q.shape[1], k.shape[1]
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, 0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, 0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    mask = torch.ones(q.shape[0], k.shape[0], dtype=torch.bool, device=q.device)
    if causal:
        mask &= k_pos[None, :] <= q_pos[:, None]
    if seg_q is not None:
        mask &= seg_q[:, None] == seg_k[None, :]
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.masked_fill(torch.isinf(lse), 0.0).unsqueeze(-1))
    o = torch.matmul(p, vf).transpose(0, 1)
    if return_lse:
        return o, lse.transpose(0, 1)
    return o.to(q.dtype)


def _positions(T_local: int, cp: int, rank: int, device, cu_seqlens=None, row_length: Optional[int] = None):
    """Positions of this rank's tokens in the concatenation of the micro-batch's full rows (every row is cut into
    2*cp chunks; rank r holds chunks r and 2cp-1-r of EACH row, see `get_batch_on_this_cp_rank`) and, for packed
    rows, the index of the sequence each token belongs to. That order is causal order inside every sequence, so masks
    built from (position, sequence) are exact for sequences of any lengths; only the row length has to divide by 2*cp."""
    total = T_local * cp
    row = row_length or total
    one = cp_chunk_indices(row, cp, rank, device)
    n_rows = total // row
    pos = one if n_rows == 1 else (one[None, :] + torch.arange(n_rows, device=device)[:, None] * row).reshape(-1)
    if cu_seqlens is None:
        if n_rows == 1:
            return pos, None
        return pos, torch.div(pos, row, rounding_mode="floor")
    seg = torch.bucketize(pos, cu_seqlens[1:].to(device=device, dtype=pos.dtype), right=True)
    return pos, seg


def gather_full_sequence(tensors, row_length: Optional[int] = None):
    """For layers whose mixing runs ALONG the sequence and cannot be cut into independent chunks (causal convolution,
    recurrent / linear attention, window + compressed attention): every context-parallel rank gathers the tensors of
    all ranks and puts the tokens into row order. Returns ``(full tensors, own)`` where ``own`` are the row positions
    of this rank's tokens, i.e. ``full_out[own]`` is the local part of a result computed on the full sequence. The
    mixing is computed redundantly on every rank; in backward the gather reduce-scatters, so each rank contributes the
    gradient of its own tokens' outputs and receives the total for its own inputs."""
    st = ps.get_state()
    cp, rank, g = st.dims.cp, st.cp_rank, st.group("cp")
    T = tensors[0].shape[0]
    own, _ = _positions(T, cp, rank, tensors[0].device, None, row_length)
    order = torch.argsort(M._all_gather_dim0(own, g))
    full = [M.gather_from_sequence_parallel_region(t.contiguous(), g, True).index_select(0, order) for t in tensors]
    return full, own


def ring_attention(q, k, v, *, causal=True, scale=None, cu_seqlens=None, row_length: Optional[int] = None):
    """Attention for sequence-sharded q/k/v ``[T/cp, H, D]`` (load-balanced chunks)."""
    st = ps.get_state()
    cp, rank, g = st.dims.cp, st.cp_rank, st.group("cp")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    kind = _CFG["comm_type"]
    Hq, Hkv = q.shape[1], k.shape[1]
    if kind == "auto":
        kind = "a2a" if (Hq % cp == 0 and Hkv % cp == 0 and cu_seqlens is None and row_length is None) else "allgather"
    if kind == "a2a":
        return _ulysses(q, k, v, causal, scale, cp, rank, g)
    pos, seg = _positions(q.shape[0], cp, rank, q.device, cu_seqlens, row_length)
    if kind == "a2a+p2p":
        # inner all-to-all: all tokens of the block's ranks, a slice of the heads; the ring then runs between the
        # blocks with explicit positions (and segment ids), so the gathered token order needs no permutation
        gi, go = st.group("cp_inner"), st.group("cp_outer")
        n_outer = len(st.ranks("cp_outer"))
        qh, kh, vh = (M.all_to_all_sp2hp(t, gi) for t in (q, k, v))
        pos_h = M._all_gather_dim0(pos, gi)
        seg_h = M._all_gather_dim0(seg, gi) if seg is not None else None
        o = _RingP2P.apply(qh, kh, vh, pos_h, seg_h, scale, causal, n_outer, st.rank_in("cp_outer"), go)
        return M.all_to_all_hp2sp(o, gi)
    if kind == "allgather":
        k_all = M.gather_from_sequence_parallel_region(k, g, True)
        v_all = M.gather_from_sequence_parallel_region(v, g, True)
        pos_all = M._all_gather_dim0(pos, g)
        seg_all = M._all_gather_dim0(seg, g) if seg is not None else None
        return _masked_attention(q, k_all, v_all, pos, pos_all, scale, causal, seg, seg_all)
    return _RingP2P.apply(q, k, v, pos, seg, scale, causal, cp, rank, g)


def _ulysses(q, k, v, causal, scale, cp, rank, g):
    """Sequence-sharded -> head-sharded, full-sequence attention, and back. The local token order is
    (chunk r, chunk 2cp-1-r); after the all-to-all the gathered order is rank-major, so tokens are
    permuted into true sequence order for the causal kernel and back afterwards."""
    T_local = q.shape[0]
    qh = M.all_to_all_sp2hp(q, g)
    kh = M.all_to_all_sp2hp(k, g)
    vh = M.all_to_all_sp2hp(v, g)
    order = torch.cat([cp_chunk_indices(T_local * cp, cp, r, q.device) for r in range(cp)])  # gathered -> position
    inv = torch.argsort(order)
    o = OF.attention(qh.index_select(0, inv), kh.index_select(0, inv), vh.index_select(0, inv), causal=causal,
                     scale=scale)
    o = o.index_select(0, order)
    return M.all_to_all_hp2sp(o, g)


class _RingP2P(torch.autograd.Function):
    """KV blocks travel around the ring; partial outputs are merged with their log-sum-exp.
    Backward recomputes block probabilities from the saved global LSE and sends dK/dV around the
    ring back to their owners."""

    @staticmethod
    def _exchange(t, g, cp, rank):
        ranks = dist.get_process_group_ranks(g)
        nxt, prv = ranks[(rank + 1) % cp], ranks[(rank - 1) % cp]
        recv = torch.empty_like(t)
        ops = [dist.P2POp(dist.isend, t.contiguous(), nxt, g), dist.P2POp(dist.irecv, recv, prv, g)]
        if rank % 2:
            ops.reverse()
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        return recv

    @staticmethod
    def forward(ctx, q, k, v, pos, seg, scale, causal, cp, rank, g):
        T = q.shape[0]
        o = torch.zeros(T, q.shape[1], v.shape[2], dtype=torch.float32, device=q.device)
        lse = torch.full((T, q.shape[1]), float("-inf"), dtype=torch.float32, device=q.device)
        kb, vb, pb, sb = k, v, pos, seg
        for step in range(cp):
            ob, lb = _masked_attention(q, kb, vb, pos, pb, scale, causal, seg, sb, return_lse=True)
            new = torch.logaddexp(lse, lb)
            w_old = torch.exp(lse - new).masked_fill(torch.isinf(new), 0.0)
            w_new = torch.exp(lb - new).masked_fill(torch.isinf(new), 0.0)
            o = o * w_old.unsqueeze(-1) + ob * w_new.unsqueeze(-1)
            lse = new
            if step < cp - 1:
                kb = _RingP2P._exchange(kb, g, cp, rank)
                vb = _RingP2P._exchange(vb, g, cp, rank)
                pb = _RingP2P._exchange(pb, g, cp, rank)
                if sb is not None:
                    sb = _RingP2P._exchange(sb, g, cp, rank)
        ctx.save_for_backward(q, k, v, pos, seg if seg is not None else pos, o, lse)
        ctx.cfg = (scale, causal, cp, rank, g, seg is not None)
        return o.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, pos, seg, o, lse = ctx.saved_tensors
        scale, causal, cp, rank, g, has_seg = ctx.cfg
        seg = seg if has_seg else None
        Hq, Hkv = q.shape[1], k.shape[1]
        rep = Hq // Hkv
        dof = do.float()
        delta = (dof * o).sum(-1)  # [T, Hq]
        dq = torch.zeros_like(q, dtype=torch.float32)
        kb, vb, pb, sb = k, v, pos, seg
        dkb = torch.zeros_like(k, dtype=torch.float32)
        dvb = torch.zeros_like(v, dtype=torch.float32)
        for step in range(cp):
            kf = kb.float().transpose(0, 1).repeat_interleave(rep, 0)
            vf = vb.float().transpose(0, 1).repeat_interleave(rep, 0)
            s = torch.matmul(q.float().transpose(0, 1), kf.transpose(1, 2)) * scale
            mask = torch.ones(q.shape[0], kb.shape[0], dtype=torch.bool, device=q.device)
            if causal:
                mask &= pb[None, :] <= pos[:, None]
            if sb is not None:
                mask &= seg[:, None] == sb[None, :]
            p = torch.exp(s - lse.transpose(0, 1).unsqueeze(-1)).masked_fill(~mask, 0.0)
            p = torch.nan_to_num(p)
            dv_h = torch.matmul(p.transpose(1, 2), dof.transpose(0, 1))  # [Hq, Tk, D]
            dp = torch.matmul(dof.transpose(0, 1), vf.transpose(1, 2))
            ds = p * (dp - delta.transpose(0, 1).unsqueeze(-1)) * scale
            dq += torch.matmul(ds, kf).transpose(0, 1)
            dk_h = torch.matmul(ds.transpose(1, 2), q.float().transpose(0, 1))
            dkb += dk_h.view(Hkv, rep, *dk_h.shape[1:]).sum(1).transpose(0, 1)
            dvb += dv_h.view(Hkv, rep, *dv_h.shape[1:]).sum(1).transpose(0, 1)
            # the gradient buffers travel with their KV block; after cp hops they are home again
            kb = _RingP2P._exchange(kb, g, cp, rank)
            vb = _RingP2P._exchange(vb, g, cp, rank)
            pb = _RingP2P._exchange(pb, g, cp, rank)
            if sb is not None:
                sb = _RingP2P._exchange(sb, g, cp, rank)
            dkb = _RingP2P._exchange(dkb, g, cp, rank)
            dvb = _RingP2P._exchange(dvb, g, cp, rank)
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None, None, None, None, None
