"""Context-parallel attention schemes against single-process attention on the full micro-batch: packed sequences
whose boundaries fall inside chunks, several rows per micro-batch, every communication type, forward and backward.
All schemes run through the same range-pair primitive that a GPU serves with the flash kernel."""
import pytest
import torch

from dist_utils import run_distributed


def _worker(rank, world, comm, cu, row, causal, heads):
    from loongforge_b200.ops import functional as OF
    from loongforge_b200.parallel import context_parallel as CP
    from loongforge_b200.parallel import state as ps

    ps.initialize_model_parallel(ps.ParallelDims(cp=world))
    if comm == "a2a+p2p":
        CP.set_cp_comm_type(comm, 2)
    else:
        CP.set_cp_comm_type(comm)
    try:
        Hq, Hkv = heads
        T, D = 96 * (2 if row else 1), 16
        torch.manual_seed(0)
        q = torch.randn(T, Hq, D, dtype=torch.float64)
        k = torch.randn(T, Hkv, D, dtype=torch.float64)
        v = torch.randn(T, Hkv, D, dtype=torch.float64)
        do = torch.randn(T, Hq, D, dtype=torch.float64)
        row_len = row or T
        # reference on the full micro-batch: rows and packed sequences are both attention boundaries
        bounds = sorted(set(range(0, T + 1, row_len)) | set(cu or []))
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        ref = OF.attention_ref(qr, kr, vr, causal, None, torch.tensor(bounds))
        ref.backward(do)
        # this rank's tokens: chunks r and 2cp-1-r of every row
        idx = torch.cat([CP.cp_chunk_indices(row_len, world, rank) + r0 for r0 in range(0, T, row_len)])
        ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
        o = CP.ring_attention(ql, kl, vl, causal=causal, cu_seqlens=torch.tensor(cu) if cu else None,
                              row_length=row)
        o.backward(do[idx])
        err = lambda a, b: float((a.detach() - b.detach()).abs().max())  # noqa: E731
        return [err(o, ref[idx].detach()), err(ql.grad, qr.grad[idx]), err(kl.grad, kr.grad[idx]),
                err(vl.grad, vr.grad[idx])]
    finally:
        CP.set_cp_comm_type("auto")


@pytest.mark.parametrize("comm", ["p2p", "allgather", "a2a"])
@pytest.mark.parametrize("cu,row", [([0, 7, 30, 31, 70, 96], None),   # packed, boundaries inside and across chunks
                                    (None, 96),                       # two rows, no packing
                                    ([0, 50, 96, 100, 192], 96)])     # two packed rows
@pytest.mark.parametrize("causal", [True, False])
def test_cp2_matches_full_attention(comm, cu, row, causal):
    for errs in run_distributed(_worker, 2, comm, cu, row, causal, (4, 2)):
        assert max(errs) < 3e-4, errs  # blocks are evaluated in fp32 (sums in another order than the reference)


@pytest.mark.parametrize("comm", ["p2p", "allgather", "a2a", "a2a+p2p"])
def test_cp4_packed_matches_full_attention(comm):
    for errs in run_distributed(_worker, 4, comm, [0, 13, 40, 41, 77, 96], None, True, (8, 4)):
        assert max(errs) < 3e-4, errs  # blocks are evaluated in fp32 (sums in another order than the reference)
