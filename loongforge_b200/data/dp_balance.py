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


def solve_assignment(lengths_per_rank: Sequence[Sequence[int]], model: CostModel,
                     capacity: int = 0) -> List[List[Tuple[int, int]]]:
    """-> for every destination rank the list of (source rank, index in source) it should process. Deterministic, so
    every rank computes the same plan from the same gathered lengths. ``capacity`` > 0 caps the number of items per
    rank (whole micro-batches are moved and every rank must keep the same micro-batch count)."""
    world = len(lengths_per_rank)
    items = [(float(model.cost([n])[0]), r, i) for r, ls in enumerate(lengths_per_rank) for i, n in enumerate(ls)]
    items.sort(key=lambda t: (-t[0], t[1], t[2]))
    load = [0.0] * world
    plan: List[List[Tuple[int, int]]] = [[] for _ in range(world)]
    for c, r, i in items:
        open_ranks = [k for k in range(world) if not capacity or len(plan[k]) < capacity]
        d = min(open_ranks, key=lambda k: (load[k], k))
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


# ----------------------------------------------------------------------------- whole micro-batches
class BalancedMicrobatchIterator:
    """Wraps a rank's micro-batch iterator: once per step (every ``num_microbatches`` pulls) the data-parallel ranks
    publish the token counts of their micro-batches, solve one assignment with the same micro-batch count per rank,
    and trade whole micro-batches so that the most expensive ones do not pile up on one rank (reference hook:
    loongforge/data/dp_balance/train_hooks.py:117-181; plan and exchange: rebalance/balance.py:275-737).

    A micro-batch is a dict of tensors (any shapes; e.g. tokens / labels / loss_mask / position_ids / cu_seqlens, pixel
    patches and their grids for VLMs) plus plain Python values, which travel with it. Integer and boolean tensors move
    as one int64 payload, floating tensors as one float32 payload: two variable-size all-to-alls per step. The
    micro-batch SET of the step is unchanged, so the step's loss and gradients are those of the unbalanced run."""

    def __init__(self, iterator, num_microbatches: int, group=None, model: CostModel = None, length_key: str = "tokens"):
        self.it, self.nmb, self.group = iterator, num_microbatches, group
        self.model = model or CostModel()
        self.length_key = length_key
        self.buffer: List[dict] = []
        self.last_imbalance = (1.0, 1.0)  # (before, after) of the latest step
        self.last_lengths: List[int] = []  # token counts of the micro-batches this rank ran in the latest step

    def __iter__(self):
        return self

    def __next__(self):
        if not self.buffer:
            self.buffer = self._exchange([next(self.it) for _ in range(self.nmb)])
            self.last_lengths = [int(b[self.length_key].numel()) for b in self.buffer]
        return self.buffer.pop(0)

    # -- (de)serialisation of one micro-batch
    @staticmethod
    def _pack(b: dict):
        meta, ints, floats, plain = [], [], [], {}
        for k, v in b.items():
            if not torch.is_tensor(v):
                plain[k] = v
                continue
            is_f = v.is_floating_point()
            meta.append((k, str(v.dtype).replace("torch.", ""), tuple(v.shape), is_f))
            (floats if is_f else ints).append(v.detach().reshape(-1).to("cpu", torch.float32 if is_f else torch.int64))
        cat = lambda xs, dt: torch.cat(xs) if xs else torch.empty(0, dtype=dt)  # noqa: E731
        return meta, plain, cat(ints, torch.int64), cat(floats, torch.float32)

    @staticmethod
    def _unpack(meta, plain, ints: torch.Tensor, floats: torch.Tensor) -> dict:
        out, oi, of = dict(plain), 0, 0
        for k, dt, shape, is_f in meta:
            n = 1
            for d in shape:
                n *= d
            if is_f:
                out[k], of = floats[of:of + n].view(shape).to(getattr(torch, dt)), of + n
            else:
                out[k], oi = ints[oi:oi + n].view(shape).to(getattr(torch, dt)), oi + n
        return out

    def _exchange(self, batches: List[dict]) -> List[dict]:
        g = self.group
        if not dist.is_initialized() or dist.get_world_size(g) == 1:
            return batches
        from ..parallel.mappings import all_to_all_single

        g = g if g is not None else dist.group.WORLD
        world, rank = dist.get_world_size(g), dist.get_rank(g)
        packed = [self._pack(b) for b in batches]
        mine = [(int(b[self.length_key].numel()), m, pl, int(i.numel()), int(f.numel()))
                for b, (m, pl, i, f) in zip(batches, packed)]
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=g)
        lengths = [[it[0] for it in r] for r in gathered]
        plan = solve_assignment(lengths, self.model, capacity=self.nmb)
        after = [[lengths[r][i] for (r, i) in plan[d]] for d in range(world)]
        self.last_imbalance = (imbalance(lengths, self.model), imbalance(after, self.model))
        send = [[i for (r, i) in plan[d] if r == rank] for d in range(world)]
        recv = [[(r, i) for (r, i) in plan[rank] if r == src] for src in range(world)]
        payloads = []
        for which, dt in ((2, torch.int64), (3, torch.float32)):
            ins = [torch.cat([packed[i][which] for i in idx]) if idx else torch.empty(0, dtype=dt) for idx in send]
            out_sizes = [sum(gathered[r][i][which + 1] for (r, i) in pairs) for pairs in recv]
            flat = torch.empty(sum(out_sizes), dtype=dt)
            dev = _comm_device(g)
            src = torch.cat(ins).to(dev)
            dst = flat.to(dev)
            all_to_all_single(dst, src, out_sizes, [int(c.numel()) for c in ins], g)
            payloads.append(dst.cpu())
        out, oi, of = [], 0, 0
        for pairs in recv:
            for (r, i) in pairs:
                _, meta, plain, ni, nf = gathered[r][i]
                out.append(self._unpack(meta, plain, payloads[0][oi:oi + ni], payloads[1][of:of + nf]))
                oi, of = oi + ni, of + nf
        return out


def _comm_device(group) -> torch.device:
    """Tensors of a collective must live where the group's backend works: the GPU for NCCL, the host for gloo."""
    backend = dist.get_backend(group)
    return torch.device("cuda", torch.cuda.current_device()) if "nccl" in str(backend) else torch.device("cpu")


def fit_cost_model_across_ranks(model: CostModel, group=None) -> np.ndarray:
    """Warm-up fit (reference: loongforge/data/dp_balance/rebalance/warmup.py:55-139): every rank has observed
    (lengths of the micro-batches it ran, its forward + backward time) for a few steps; the observations of all ranks
    are pooled so that every rank fits, and from then on plans with, the same coefficients."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        pooled: List[list] = [None] * dist.get_world_size(group)
        dist.all_gather_object(pooled, model.obs, group=group)
        model.obs = [o for part in pooled for o in part]
    return model.fit()
