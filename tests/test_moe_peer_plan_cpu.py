"""Index arithmetic of the peer-memory MoE dispatcher, emulated on CPU for two expert-parallel ranks:
push lands every (token, expert) pair in an expert-sorted row of the owning rank, pull sums them back."""
import torch

from loongforge_b200.parallel.moe_peer import RoutePlan


def test_route_plan_push_pull_roundtrip():
    torch.manual_seed(0)
    ep, E, k, H = 2, 8, 3, 16
    El = E // ep
    Ts = [13, 9]
    xs = [torch.randn(T, H) for T in Ts]
    idx = [torch.stack([torch.randperm(E)[:k] for _ in range(T)]) for T in Ts]
    counts = torch.stack([torch.bincount(i.reshape(-1), minlength=E) for i in idx])
    plans = [RoutePlan(idx[r], E, ep, r, None, 10_000, all_counts=counts) for r in range(ep)]
    cap = max(sum(p.tokens_per_expert) for p in plans)
    bufs = [torch.full((cap, H), float("nan")) for _ in range(ep)]
    owner = [torch.full((cap,), -1, dtype=torch.long) for _ in range(ep)]
    for r, p in enumerate(plans):
        for j in range(p.pair_token.numel()):
            d, row = int(p.pair_dst[j]), int(p.pair_row[j])
            assert owner[d][row] == -1, "two pairs landed on one row"
            bufs[d][row] = xs[r][int(p.pair_token[j])]
            owner[d][row] = int(p.pair_expert[j])
    for d, p in enumerate(plans):
        rows = sum(p.tokens_per_expert)
        assert p.rows == rows and not torch.isnan(bufs[d][:rows]).any()
        # rows are sorted by local expert with the announced counts
        expect = torch.repeat_interleave(torch.arange(El) + d * El, torch.tensor(p.tokens_per_expert))
        assert torch.equal(owner[d][:rows], expect)
        assert p.tokens_per_expert == counts[:, d * El:(d + 1) * El].sum(0).tolist()
    # experts scale rows by (expert id + 1); pull must return sum_k (e_k + 1) * x[t]
    ys = [b * (o.clamp(min=0) + 1).unsqueeze(-1) for b, o in zip(bufs, owner)]
    for r, p in enumerate(plans):
        out = torch.zeros(Ts[r], H)
        for t in range(Ts[r]):
            for kk in range(k):
                j = int(p.slot_pair[t * k + kk])
                assert int(p.pair_token[j]) == t
                out[t] += ys[int(p.pair_dst[j])][int(p.pair_row[j])]
        ref = xs[r] * (idx[r] + 1).sum(-1, keepdim=True)
        assert torch.allclose(out, ref, atol=1e-5)
