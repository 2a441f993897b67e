"""Context parallelism: load-balanced sequence sharding of the batch and three attention
communication schemes.

* ``get_batch_on_this_cp_rank`` / ``cp_chunk_indices``: each sequence is cut into ``2*cp`` chunks and
  rank r keeps chunks ``r`` and ``2*cp-1-r`` (causal load balance), the input preparation the
  reference does in loongforge/models/omni_models/utils.py:26-184 and
  loongforge/train/pretrain/pretrain_llm.py:70.
* ``cp_comm_type`` (every scheme runs its attention through the flash kernel, O(T) memory per step):
    - ``"p2p"``      ring of KV chunks, a few kernel calls per step merged by their log-sum-exp;
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


# ----------------------------------------------------------------------------- attention on sequence chunks
# Every scheme below is built from ONE primitive: the attention of a contiguous range of query positions against a
# contiguous range of key positions of the same micro-batch, through `ops.functional.attention_with_lse` (the tcgen05
# flash kernel on a GPU, its fp32 formulation on CPU), which returns the log-sum-exp that partial results are merged
# with. Memory stays O(T) per step. Packed sequences and several rows per micro-batch become sequence boundaries
# ("segments") that are clipped to the two ranges on the host; a causal mask is always expressed as the kernel's
# bottom-right aligned mask of a (query part, key part) pair that ends at the same position.

_HOST_CU: Dict[tuple, list] = {}


def _host_boundaries(cu_seqlens) -> Optional[list]:
    """Sequence boundaries as Python ints. The device-to-host read happens once per tensor (all layers of a
    micro-batch pass the same one)."""
    if cu_seqlens is None:
        return None
    if isinstance(cu_seqlens, (list, tuple)):
        return [int(x) for x in cu_seqlens]
    key = (cu_seqlens.data_ptr(), cu_seqlens.numel(), cu_seqlens._version, str(cu_seqlens.device))
    hit = _HOST_CU.get(key)
    if hit is None:
        if len(_HOST_CU) > 64:
            _HOST_CU.clear()
        hit = _HOST_CU[key] = [int(x) for x in cu_seqlens.tolist()]
    return hit


def _segments(total: int, row: int, cu: Optional[list]) -> list:
    """[a, b) position ranges inside which tokens may attend to each other: the packed sequences, cut at the rows of
    the micro-batch (positions count through the concatenation of the rows)."""
    bounds = set(range(0, total, row)) | {total}
    if cu:
        bounds |= {x for x in cu if 0 <= x <= total}
    bs = sorted(bounds)
    return list(zip(bs[:-1], bs[1:]))


def _clip(segs, q_lo, q_hi, k_lo, k_hi):
    """Boundary lists (relative to q_lo and to the first used key) of the segments that hold queries of [q_lo, q_hi),
    with their keys inside [k_lo, k_hi). Returns (cu_q, cu_k, k_first) or None when no query sees any key."""
    cu_q, cu_k, k_first = [0], [0], None
    for a, b in segs:
        qa, qb = max(a, q_lo), min(b, q_hi)
        if qa >= qb:
            continue
        ka, kb = max(a, k_lo), min(b, k_hi)
        cu_q.append(qb - q_lo)
        if ka >= kb:
            cu_k.append(cu_k[-1])
            continue
        if k_first is None:
            k_first = ka
        assert ka - k_first == cu_k[-1], "key parts of consecutive segments must be contiguous"
        cu_k.append(kb - k_first)
    if k_first is None:
        return None
    return cu_q, cu_k, k_first


def _range_call(segs, q_lo, q_hi, k_lo, k_hi, k_base):
    """Arguments of the kernel call for queries [q_lo, q_hi) x keys [k_lo, k_hi) of a key tensor whose row 0 is
    position `k_base`: (key slice start, key slice end, cu_q, cu_k) or None. The boundary lists are dropped when a
    single segment covers both ranges."""
    c = _clip(segs, q_lo, q_hi, k_lo, k_hi)
    if c is None:
        return None
    cu_q, cu_k, k_first = c
    ks, ke = k_first - k_base, k_first - k_base + cu_k[-1]
    if len(cu_q) == 2:
        return ks, ke, None, None
    return ks, ke, cu_q, cu_k


def _cu_tensor(lst, device):
    return None if lst is None else torch.tensor(lst, dtype=torch.int32, device=device)


def _merge(o, lse, ob, lb):
    """Online-softmax merge of a partial result (ob bf16/fp32 [T, H, D], lb [H, T]) into the fp32 running pair."""
    new = torch.logaddexp(lse, lb)
    dead = torch.isinf(new) & (new < 0)
    w_old = torch.exp(lse - new).masked_fill(dead, 0.0).t().unsqueeze(-1)
    w_new = torch.exp(lb - new).masked_fill(dead, 0.0).t().unsqueeze(-1)
    return o * w_old + ob.float() * w_new, new


class _ChunkLayout:
    """Where the tokens of a (ring size n, ring rank r) participant sit: per row of the micro-batch two chunks of
    length L, chunk r and chunk 2n-1-r (load-balanced for causal masks); local order is [row][early, late][L]."""

    def __init__(self, t_local: int, n: int, r: int, row_length: Optional[int]):
        total = t_local * n
        self.row = row_length or total
        self.n, self.r, self.total = n, r, total
        self.n_rows = total // self.row
        self.L = self.row // (2 * n)
        assert self.L * 2 * n == self.row, "row length must divide by 2 * context-parallel size"

    def chunks(self, r: Optional[int] = None):
        """(local offset, global position) of every chunk held by ring rank r (default: this one)."""
        r = self.r if r is None else r
        out = []
        for i in range(self.n_rows):
            out.append((i * 2 * self.L, i * self.row + r * self.L))
            out.append((i * 2 * self.L + self.L, i * self.row + (2 * self.n - 1 - r) * self.L))
        return out


def _attend_chunks(q, k, v, lay: _ChunkLayout, k_rank: int, segs, causal, scale, acc):
    """All (query chunk of this rank) x (key chunk held by ring rank `k_rank`, passed as k / v) pairs that see each
    other; results are merged into acc = (o fp32, lse)."""
    o, lse = acc
    L = lay.L
    for q_off, q_pos in lay.chunks():
        for k_off, k_pos in lay.chunks(k_rank):
            if q_pos // lay.row != k_pos // lay.row:
                continue  # different rows never attend to each other
            if causal and k_pos > q_pos:
                continue
            call = _range_call(segs, q_pos, q_pos + L, k_pos, k_pos + L, k_pos - k_off)
            if call is None:
                continue
            ks, ke, cu_q, cu_k = call
            ob, lb = OF.attention_with_lse(q[q_off:q_off + L], k[ks:ke], v[ks:ke], causal=causal and k_pos == q_pos,
                                           scale=scale, cu_seqlens=_cu_tensor(cu_q, q.device),
                                           cu_seqlens_k=_cu_tensor(cu_k, q.device))
            o[q_off:q_off + L], lse[:, q_off:q_off + L] = _merge(o[q_off:q_off + L], lse[:, q_off:q_off + L], ob, lb)
    return o, lse


def _attend_chunks_bwd(do, q, k, v, o, lse, lay, k_rank, segs, causal, scale, dq, dk, dv):
    """Gradient contributions of the same pairs: dq accumulates locally, dk / dv into the buffers that travel with
    the key chunk. `o` / `lse` are the final (merged) forward results."""
    L = lay.L
    for q_off, q_pos in lay.chunks():
        for k_off, k_pos in lay.chunks(k_rank):
            if q_pos // lay.row != k_pos // lay.row or (causal and k_pos > q_pos):
                continue
            call = _range_call(segs, q_pos, q_pos + L, k_pos, k_pos + L, k_pos - k_off)
            if call is None:
                continue
            ks, ke, cu_q, cu_k = call
            sl = slice(q_off, q_off + L)
            g = _pair_backward(do[sl], q[sl], k[ks:ke], v[ks:ke], o[sl], lse[:, sl].contiguous(), cu_q, cu_k, scale,
                               causal and k_pos == q_pos)
            dq[sl] += g[0].float()
            dk[ks:ke] += g[1].float()
            dv[ks:ke] += g[2].float()


def _pair_backward(do, q, k, v, o, lse, cu_q, cu_k, scale, causal):
    """(dq, dk, dv) of one range pair against the given (merged) output and log-sum-exp."""
    if q.is_cuda and OF.native_attention_supported(q, k, v):
        return OF.attention_backward(do.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), o.contiguous(),
                                     lse, _cu_tensor(cu_q, q.device), _cu_tensor(cu_k, q.device), scale, causal)
    # fp32 formulation (CPU): probabilities from the merged lse, as the kernels do
    Hq, Hkv = q.shape[1], k.shape[1]
    rep = Hq // Hkv
    qf, kf, vf = q.float().transpose(0, 1), k.float().transpose(0, 1), v.float().transpose(0, 1)
    kr, vr = kf.repeat_interleave(rep, 0), vf.repeat_interleave(rep, 0)
    s = torch.matmul(qf, kr.transpose(1, 2)) * scale
    seg_q, pos_q, len_q = OF._seq_ids(q.shape[0], _cu_tensor(cu_q, q.device), q.device)
    seg_k, pos_k, len_k = OF._seq_ids(k.shape[0], _cu_tensor(cu_k, q.device), q.device)
    mask = seg_q[:, None] == seg_k[None, :]
    if causal:
        mask &= pos_k[None, :] <= (pos_q + (len_k - len_q)[seg_q])[:, None]
    pr = torch.exp(s - lse.unsqueeze(-1)).masked_fill(~mask, 0.0)
    pr = torch.nan_to_num(pr, nan=0.0, posinf=0.0)
    dof = do.float().transpose(0, 1)
    delta = (do.float() * o.float()).sum(-1).t().unsqueeze(-1)
    dvh = torch.matmul(pr.transpose(1, 2), dof)
    ds = pr * (torch.matmul(dof, vr.transpose(1, 2)) - delta) * scale
    dq = torch.matmul(ds, kr).transpose(0, 1)
    dkh = torch.matmul(ds.transpose(1, 2), qf)
    dk = dkh.view(Hkv, rep, *dkh.shape[1:]).sum(1).transpose(0, 1)
    dv = dvh.view(Hkv, rep, *dvh.shape[1:]).sum(1).transpose(0, 1)
    return dq, dk, dv


def ring_attention(q, k, v, *, causal=True, scale=None, cu_seqlens=None, row_length: Optional[int] = None):
    """Attention for sequence-sharded q/k/v ``[T/cp, H, D]`` (load-balanced chunks)."""
    st = ps.get_state()
    cp, rank, g = st.dims.cp, st.cp_rank, st.group("cp")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    kind = _CFG["comm_type"]
    Hq, Hkv = q.shape[1], k.shape[1]
    if kind == "auto":
        kind = "a2a" if (Hq % cp == 0 and Hkv % cp == 0) else "allgather"
    lay = _ChunkLayout(q.shape[0], cp, rank, row_length)
    segs = _segments(lay.total, lay.row, _host_boundaries(cu_seqlens))
    if kind == "a2a":
        return _ulysses(q, k, v, causal, scale, lay, segs, g)
    if kind == "a2a+p2p":
        # inner all-to-all: all tokens of the block's ranks, a slice of the heads. The u neighbouring ranks of a block
        # hold two runs of u consecutive chunks, i.e. two chunks of length u*L of a ring of cp/u participants.
        gi, go = st.group("cp_inner"), st.group("cp_outer")
        u, n_outer = len(st.ranks("cp_inner")), len(st.ranks("cp_outer"))
        perm = _inner_block_order(lay, u, q.device)
        qh, kh, vh = (M.all_to_all_sp2hp(t, gi).index_select(0, perm) for t in (q, k, v))
        big = _ChunkLayout(qh.shape[0], n_outer, st.rank_in("cp_outer"), row_length)
        o = _RingP2P.apply(qh, kh, vh, scale, causal, big, segs, go)
        return M.all_to_all_hp2sp(o.index_select(0, torch.argsort(perm)), gi)
    if kind == "allgather":
        return _AllGatherKV.apply(q, k, v, scale, causal, lay, segs, g)
    return _RingP2P.apply(q, k, v, scale, causal, lay, segs, g)


def _inner_block_order(lay: _ChunkLayout, u: int, device) -> torch.Tensor:
    """Permutation from the inner all-to-all's token order ([inner rank][row][early, late][L]) to the chunk layout of
    the outer ring ([row][early, late][u * L]): the early run ascends with the inner rank, the late run descends."""
    L, rows = lay.L, lay.n_rows
    src = torch.arange(u * rows * 2 * L, device=device).view(u, rows, 2, L)
    early = src[:, :, 0].permute(1, 0, 2)                   # [row][i][L]
    late = src[:, :, 1].flip(0).permute(1, 0, 2)            # [row][u-1-i][L]
    return torch.stack([early, late], dim=1).reshape(-1)


def _ulysses(q, k, v, causal, scale, lay: _ChunkLayout, segs, g):
    """Sequence-sharded -> head-sharded, full-sequence attention, and back. After the all-to-all the gathered order
    is rank-major, so tokens are permuted into position order for the kernel and back afterwards; packed sequences
    and the rows of a multi-row micro-batch are handed to the kernel as sequence boundaries."""
    cp = lay.n
    qh = M.all_to_all_sp2hp(q, g)
    kh = M.all_to_all_sp2hp(k, g)
    vh = M.all_to_all_sp2hp(v, g)
    order = torch.cat([_positions(q.shape[0], cp, r, q.device, None, lay.row)[0] for r in range(cp)])
    inv = torch.argsort(order)  # position -> gathered index
    cu = None
    if len(segs) > 1:
        cu = torch.tensor([0] + [b for _, b in segs], dtype=torch.int32, device=q.device)
    o = OF.attention(qh.index_select(0, inv), kh.index_select(0, inv), vh.index_select(0, inv), causal=causal,
                     scale=scale, cu_seqlens=cu)
    o = o.index_select(0, order)
    return M.all_to_all_hp2sp(o, g)


class _AllGatherKV(torch.autograd.Function):
    """K / V all-gathered once over NVLink (cheap next to the attention itself: GQA keys are small), every local query
    chunk then attends to its causal prefix of the gathered sequence in one kernel call. Backward re-gathers K / V
    instead of keeping them, and reduce-scatters dK / dV."""

    @staticmethod
    def _gathered(k, v, lay, g):
        order = torch.cat([_positions(k.shape[0], lay.n, r, k.device, None, lay.row)[0] for r in range(lay.n)])
        inv = torch.argsort(order)
        ks = M._all_gather_dim0(k, g).index_select(0, inv)
        vs = M._all_gather_dim0(v, g).index_select(0, inv)
        return ks, vs, order

    @staticmethod
    def _calls(lay, segs, causal):
        for q_off, q_pos in lay.chunks():
            row0 = (q_pos // lay.row) * lay.row
            k_hi = q_pos + lay.L if causal else row0 + lay.row
            call = _range_call(segs, q_pos, q_pos + lay.L, row0, k_hi, 0)
            if call is not None:
                yield q_off, call

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, lay, segs, g):
        ks, vs, _ = _AllGatherKV._gathered(k, v, lay, g)
        o = torch.zeros_like(q)
        lse = torch.full((q.shape[1], q.shape[0]), float("-inf"), dtype=torch.float32, device=q.device)
        L = lay.L
        for q_off, (a, b, cu_q, cu_k) in _AllGatherKV._calls(lay, segs, causal):
            ob, lb = OF.attention_with_lse(q[q_off:q_off + L], ks[a:b], vs[a:b], causal=causal, scale=scale,
                                           cu_seqlens=_cu_tensor(cu_q, q.device),
                                           cu_seqlens_k=_cu_tensor(cu_k, q.device))
            o[q_off:q_off + L] = ob
            lse[:, q_off:q_off + L] = lb
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (scale, causal, lay, segs, g)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, lay, segs, g = ctx.cfg
        ks, vs, order = _AllGatherKV._gathered(k, v, lay, g)
        dq = torch.zeros_like(q)
        dks = torch.zeros(ks.shape, dtype=torch.float32, device=q.device)
        dvs = torch.zeros(vs.shape, dtype=torch.float32, device=q.device)
        L = lay.L
        for q_off, (a, b, cu_q, cu_k) in _AllGatherKV._calls(lay, segs, causal):
            sl = slice(q_off, q_off + L)
            gq, gk, gv = _pair_backward(do[sl], q[sl], ks[a:b], vs[a:b], o[sl], lse[:, sl].contiguous(), cu_q, cu_k,
                                        scale, causal)
            dq[sl] = gq.to(dq.dtype)
            dks[a:b] += gk.float()
            dvs[a:b] += gv.float()
        # back to the gathered (rank-major) order, then every rank keeps the sum of its own tokens' gradients
        dk = M._reduce_scatter_dim0(dks.index_select(0, order), g)
        dv = M._reduce_scatter_dim0(dvs.index_select(0, order), g)
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None


class _RingP2P(torch.autograd.Function):
    """KV chunks travel around the ring; every step is a handful of kernel calls on (query chunk, key chunk) pairs
    (full, causal-diagonal or skipped) whose results are merged by their log-sum-exp. Backward recomputes the
    probabilities from the merged log-sum-exp and sends dK / dV around the ring with their chunks."""

    @staticmethod
    def _exchange(t, g, n, rank):
        ranks = dist.get_process_group_ranks(g)
        nxt, prv = ranks[(rank + 1) % n], ranks[(rank - 1) % n]
        recv = torch.empty_like(t)
        ops = [dist.P2POp(dist.isend, t.contiguous(), nxt, g), dist.P2POp(dist.irecv, recv, prv, g)]
        if rank % 2:
            ops.reverse()
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        return recv

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, lay, segs, g):
        n, rank = lay.n, lay.r
        T = q.shape[0]
        acc = (torch.zeros(T, q.shape[1], v.shape[2], dtype=torch.float32, device=q.device),
               torch.full((q.shape[1], T), float("-inf"), dtype=torch.float32, device=q.device))
        kb, vb = k, v
        for step in range(n):
            acc = _attend_chunks(q, kb, vb, lay, (rank - step) % n, segs, causal, scale, acc)
            if step < n - 1:
                kb = _RingP2P._exchange(kb, g, n, rank)
                vb = _RingP2P._exchange(vb, g, n, rank)
        o = acc[0].to(q.dtype)
        ctx.save_for_backward(q, k, v, o, acc[1])
        ctx.cfg = (scale, causal, lay, segs, g)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, lay, segs, g = ctx.cfg
        n, rank = lay.n, lay.r
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        kb, vb = k, v
        dkb = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
        dvb = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
        for step in range(n):
            _attend_chunks_bwd(do, q, kb, vb, o, lse, lay, (rank - step) % n, segs, causal, scale, dq, dkb, dvb)
            # the gradient buffers travel with their KV chunk; after n hops they are home again
            if step < n - 1:
                kb = _RingP2P._exchange(kb, g, n, rank)
                vb = _RingP2P._exchange(vb, g, n, rank)
            dkb = _RingP2P._exchange(dkb, g, n, rank)
            dvb = _RingP2P._exchange(dvb, g, n, rank)
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None, None, None
