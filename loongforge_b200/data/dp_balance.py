"""Data-parallel load balancing for variable-length (VLM / SFT) batches.

Per-sample cost is modelled as ``a * s^2 + b * s + c`` in the sequence length ``s`` (attention + linear + fixed);
the coefficients are fitted from measured step times during warm-up. Each step every DP rank publishes its sample
lengths, all ranks solve the same assignment (longest-processing-time greedy onto the least-loaded rank) and the
samples move with one variable-size all-to-all (reference: loongforge/data/dp_balance/train_hooks.py:117-181,
rebalance/warmup.py:55-139, rebalance/balance.py:275-737, vit_balance.py:27-155)."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


class CostModel:
    def __init__(self, a: float = 1e-6, b: float = 1e-3, c: float = 0.0):
        self.coef = np.array([a, b, c], dtype=np.float64)
        self.obs: List[Tuple[List[int], float]] = []

    def cost(self, lengths) -> np.ndarray:
        s = np.asarray(lengths, dtype=np.float64)
        return self.coef[0] * s * s + self.coef[1] * s + self.coef[2]

    def observe(self, lengths: Sequence[int], step_ms: float) -> None:
        self.obs.append((list(lengths), float(step_ms)))

    def fit(self) -> np.ndarray:
        """Least squares on (sum s^2, sum s, count) -> time, coefficients clipped at zero."""
        if len(self.obs) >= 3:
            A = np.array([[sum(x * x for x in ls), sum(ls), len(ls)] for ls, _ in self.obs], dtype=np.float64)
            y = np.array([t for _, t in self.obs])
            sol, *_ = np.linalg.lstsq(A, y, rcond=None)
            self.coef = np.clip(sol, 0.0, None)
        return self.coef


def solve_assignment(lengths_per_rank: Sequence[Sequence[int]], model: CostModel) -> List[List[Tuple[int, int]]]:
    """-> for every destination rank the list of (source rank, index in source) it should process. Deterministic, so
    every rank computes the same plan from the same gathered lengths."""
    world = len(lengths_per_rank)
    items = [(float(model.cost([n])[0]), r, i) for r, ls in enumerate(lengths_per_rank) for i, n in enumerate(ls)]
    items.sort(key=lambda t: (-t[0], t[1], t[2]))
    load = [0.0] * world
    plan: List[List[Tuple[int, int]]] = [[] for _ in range(world)]
    for c, r, i in items:
        d = min(range(world), key=lambda k: (load[k], k))
        plan[d].append((r, i))
        load[d] += c
    for p in plan:
        p.sort()
    return plan


def imbalance(lengths_per_rank, model: CostModel) -> float:
    loads = [float(model.cost(ls).sum()) if len(ls) else 0.0 for ls in lengths_per_rank]
    return max(loads) / max(np.mean(loads), 1e-12)


def rebalance(samples: List[torch.Tensor], model: CostModel, group=None) -> List[torch.Tensor]:
    """`samples`: this rank's 1-D token tensors (same dtype on all ranks). Returns the samples this rank should process
    after balancing. One all-gather of lengths + one all-to-all of tokens."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return samples
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    mine = [int(s.numel()) for s in samples]
    gathered: List[List[int]] = [None] * world
    dist.all_gather_object(gathered, mine, group=group)
    plan = solve_assignment(gathered, model)
    send = [[i for (r, i) in plan[d] if r == rank] for d in range(world)]
    dtype, dev = samples[0].dtype if samples else torch.long, samples[0].device if samples else torch.device("cpu")
    in_chunks = [torch.cat([samples[i] for i in idx]) if idx else torch.empty(0, dtype=dtype, device=dev) for idx in send]
    recv_lens = [[gathered[r][i] for (r, i) in plan[rank] if r == src] for src in range(world)]
    from ..parallel.mappings import all_to_all_single  # NCCL on GPUs, emulated with p2p on gloo

    out_sizes = [sum(ls) for ls in recv_lens]
    flat_out = torch.empty(sum(out_sizes), dtype=dtype, device=dev)
    all_to_all_single(flat_out, torch.cat(in_chunks), out_sizes, [int(c.numel()) for c in in_chunks], group)
    out_chunks = list(flat_out.split(out_sizes))
    out = []
    for chunk, ls in zip(out_chunks, recv_lens):
        out += list(chunk.split(ls)) if ls else []
    return out


def balance_vit_images(patch_counts_per_rank: Sequence[Sequence[int]]) -> List[List[Tuple[int, int]]]:
    """Encoder-level balance: images are spread so that every rank encodes a similar number of patches (cost linear in
    patches for windowed attention)."""
    return solve_assignment(patch_counts_per_rank, CostModel(0.0, 1.0, 0.0))
