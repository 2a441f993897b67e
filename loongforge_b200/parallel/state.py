"""Process-group topology: TP / CP / EP / DP / PP meshes, with named snapshots for
heterogeneous (encoder vs decoder) parallelism.

Rank order is ``tp-cp-ep-dp-pp`` (TP fastest), as in the reference
(loongforge/train/initialize.py:164-173). Several named states can coexist (one per model
component); ``change_parallel_state(name)`` switches the one that the accessor functions read,
which is how a ViT with TP=1 and an LLM with TP=2 share one job
(loongforge/train/initialize.py:96-113,136-174).

Expert parallelism follows Megatron's convention: the expert mesh is laid over the same ranks
as ``tp x cp x dp`` of a pipeline stage, as ``etp x ep x edp``.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


@dataclasses.dataclass
class ParallelDims:
    tp: int = 1
    cp: int = 1
    ep: int = 1
    pp: int = 1
    etp: int = 1  # expert tensor parallel
    vpp: Optional[int] = None  # virtual pipeline stages per rank

    def dp(self, world: int) -> int:
        denom = self.tp * self.cp * self.pp
        assert world % denom == 0, f"world {world} not divisible by tp*cp*pp={denom}"
        return world // denom


class ParallelState:
    """All process groups of one model component."""

    def __init__(self, name: str, dims: ParallelDims, world_size: int, rank: int, *, create_groups: bool = True,
                 backend: Optional[str] = None, gloo_groups: bool = False, rank_offset: int = 0):
        self.name = name
        self.dims = dims
        self.world_size = world_size
        self.rank = rank
        tp, cp, pp = dims.tp, dims.cp, dims.pp
        dp = dims.dp(world_size)
        self.dp_size = dp
        # coordinates, tp fastest
        r = rank - rank_offset
        self.tp_rank = r % tp
        self.cp_rank = (r // tp) % cp
        self.dp_rank = (r // (tp * cp)) % dp
        self.pp_rank = r // (tp * cp * dp)
        # expert mesh over the tp*cp*dp ranks of one stage
        stage = tp * cp * dp
        ep, etp = dims.ep, dims.etp
        assert stage % (ep * etp) == 0, f"tp*cp*dp={stage} not divisible by ep*etp={ep * etp}"
        self.edp_size = stage // (ep * etp)
        rs = r % stage
        self.etp_rank = rs % etp
        self.ep_rank = (rs // etp) % ep
        self.edp_rank = rs // (etp * ep)
        self.groups: Dict[str, Optional[dist.ProcessGroup]] = {}
        self.group_ranks: Dict[str, List[int]] = {}
        self.gloo: Dict[str, Optional[dist.ProcessGroup]] = {}
        if create_groups:
            self._create(backend, gloo_groups, rank_offset)

    # ------------------------------------------------------------------ construction
    def _all_rank_lists(self, rank_offset: int) -> Dict[str, List[List[int]]]:
        d = self.dims
        tp, cp, pp, dp = d.tp, d.cp, d.pp, self.dp_size
        ep, etp, edp = d.ep, d.etp, self.edp_size
        stage = tp * cp * dp

        def rk(t, c, dd, p):
            return rank_offset + t + tp * (c + cp * (dd + dp * p))

        out: Dict[str, List[List[int]]] = {k: [] for k in
                                            ("tp", "cp", "dp", "dp_cp", "pp", "mp", "tp_cp", "ep", "etp", "edp",
                                             "tp_ep", "embd", "pos_embd")}
        for p in range(pp):
            for dd in range(dp):
                for c in range(cp):
                    out["tp"].append([rk(t, c, dd, p) for t in range(tp)])
            for dd in range(dp):
                for t in range(tp):
                    out["cp"].append([rk(t, c, dd, p) for c in range(cp)])
                out["tp_cp"].append([rk(t, c, dd, p) for c in range(cp) for t in range(tp)])
            for c in range(cp):
                for t in range(tp):
                    out["dp"].append([rk(t, c, dd, p) for dd in range(dp)])
            for t in range(tp):
                out["dp_cp"].append([rk(t, c, dd, p) for dd in range(dp) for c in range(cp)])
            base = rank_offset + p * stage
            for e2 in range(edp):
                for e1 in range(ep):
                    out["etp"].append([base + t + etp * (e1 + ep * e2) for t in range(etp)])
                for t in range(etp):
                    out["ep"].append([base + t + etp * (e1 + ep * e2) for e1 in range(ep)])
                out["tp_ep"].append([base + t + etp * (e1 + ep * e2) for e1 in range(ep) for t in range(etp)])
            for e1 in range(ep):
                for t in range(etp):
                    out["edp"].append([base + t + etp * (e1 + ep * e2) for e2 in range(edp)])
        for dd in range(dp):
            for c in range(cp):
                for t in range(tp):
                    ranks = [rk(t, c, dd, p) for p in range(pp)]
                    out["pp"].append(ranks)
                    # first and last stage share the (tied) embedding gradients
                    out["embd"].append(sorted(set([ranks[0], ranks[-1]])))
                    out["pos_embd"].append([ranks[0]])
        for dd in range(dp):
            for c in range(cp):
                out["mp"].append([rk(t, c, dd, p) for p in range(pp) for t in range(tp)])
        return out

    def _create(self, backend, gloo_groups, rank_offset):
        lists = self._all_rank_lists(rank_offset)
        for kind, groups in lists.items():
            mine = None
            for ranks in groups:
                if len(ranks) == 1 or not dist.is_initialized():
                    g = None
                else:
                    g = dist.new_group(ranks, backend=backend)
                if self.rank in ranks:
                    self.groups[kind] = g
                    self.group_ranks[kind] = ranks
                    mine = ranks
            if mine is None:
                self.groups[kind] = None
                self.group_ranks[kind] = [self.rank]
        if gloo_groups and dist.is_initialized():
            for kind in ("dp", "dp_cp", "tp"):
                mine = None
                for ranks in lists[kind]:
                    g = dist.new_group(ranks, backend="gloo") if len(ranks) > 1 else None
                    if self.rank in ranks:
                        mine = g
                self.gloo[kind] = mine

    def create_hierarchical_cp_groups(self, inner: int, rank_offset: int = 0) -> None:
        """Two-level context parallelism: every context-parallel group of size cp is cut into cp / inner blocks of
        `inner` consecutive ranks ("cp_inner": Ulysses all-to-all, the ranks closest to one another) and `inner`
        strided sets of cp / inner ranks ("cp_outer": the KV ring). Collective: every rank of the job calls it."""
        cp = self.dims.cp
        if inner < 1 or cp % inner:
            raise ValueError(f"context parallel size {cp} must divide by the inner (Ulysses) degree {inner}")
        backend = dist.get_backend() if dist.is_initialized() else None
        for kind, make in (("cp_inner", lambda r: [r[b * inner:(b + 1) * inner] for b in range(cp // inner)]),
                           ("cp_outer", lambda r: [r[i::inner] for i in range(inner)])):
            self.groups[kind], self.group_ranks[kind] = None, [self.rank]
            for ranks in self._all_rank_lists(rank_offset)["cp"]:
                for sub in make(ranks):
                    g = dist.new_group(sub, backend=backend) if (len(sub) > 1 and dist.is_initialized()) else None
                    if self.rank in sub:
                        self.groups[kind], self.group_ranks[kind] = g, sub

    # ------------------------------------------------------------------ accessors
    def group(self, kind: str):
        return self.groups.get(kind)

    def ranks(self, kind: str) -> List[int]:
        return self.group_ranks.get(kind, [self.rank])

    def size(self, kind: str) -> int:
        return len(self.ranks(kind))

    def rank_in(self, kind: str) -> int:
        return self.ranks(kind).index(self.rank)

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.dims.pp - 1

    def pp_next(self) -> int:
        r = self.ranks("pp")
        return r[(self.pp_rank + 1) % len(r)]

    def pp_prev(self) -> int:
        r = self.ranks("pp")
        return r[(self.pp_rank - 1) % len(r)]


_STATES: Dict[str, ParallelState] = {}
_CURRENT: Optional[str] = None

DEFAULT_STATE = "text_decoder"


def initialize_model_parallel(dims: ParallelDims, *, name: str = DEFAULT_STATE, backend: Optional[str] = None,
                              gloo_groups: bool = False, world_size: Optional[int] = None,
                              rank: Optional[int] = None) -> ParallelState:
    """Create (and make current) the process groups of component `name`."""
    global _CURRENT
    if world_size is None:
        world_size = dist.get_world_size() if dist.is_initialized() else 1
    if rank is None:
        rank = dist.get_rank() if dist.is_initialized() else 0
    st = ParallelState(name, dims, world_size, rank, backend=backend, gloo_groups=gloo_groups)
    _STATES[name] = st
    if _CURRENT is None or name == DEFAULT_STATE:
        _CURRENT = name
    return st


def create_parallel_state(name: str, dims: ParallelDims, **kw) -> ParallelState:
    """Extra named state for an encoder with its own TP degree (must divide the decoder's TP)."""
    base = _STATES.get(DEFAULT_STATE)
    if base is not None:
        assert base.dims.tp % dims.tp == 0, "encoder TP must divide decoder TP"
    cur = _CURRENT
    st = initialize_model_parallel(dims, name=name, **kw)
    _set_current(cur)
    return st


def _set_current(name: Optional[str]):
    global _CURRENT
    _CURRENT = name


def change_parallel_state(name: str) -> str:
    """Switch the state read by the accessors; returns the previous name."""
    assert name in _STATES, f"unknown parallel state {name!r}; known: {list(_STATES)}"
    prev = _CURRENT
    _set_current(name)
    return prev


def get_state(name: Optional[str] = None) -> ParallelState:
    n = name or _CURRENT
    if n is None or n not in _STATES:
        # single-process default so that layers work without any initialisation
        initialize_model_parallel(ParallelDims(), name=DEFAULT_STATE, world_size=1, rank=0)
        n = DEFAULT_STATE
    return _STATES[n]


def destroy_model_parallel():
    global _CURRENT
    _STATES.clear()
    _CURRENT = None


def model_parallel_is_initialized() -> bool:
    return bool(_STATES)


# Megatron-style accessors ---------------------------------------------------------
def get_tensor_model_parallel_group(): return get_state().group("tp")
def get_tensor_model_parallel_world_size(): return get_state().dims.tp
def get_tensor_model_parallel_rank(): return get_state().tp_rank
def get_context_parallel_group(): return get_state().group("cp")
def get_context_parallel_world_size(): return get_state().dims.cp
def get_context_parallel_rank(): return get_state().cp_rank
def get_data_parallel_group(with_context_parallel: bool = False):
    return get_state().group("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_world_size(with_context_parallel: bool = False):
    return get_state().size("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_rank(with_context_parallel: bool = False):
    return get_state().rank_in("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_group_gloo(): return get_state().gloo.get("dp")
def get_pipeline_model_parallel_group(): return get_state().group("pp")
def get_pipeline_model_parallel_world_size(): return get_state().dims.pp
def get_pipeline_model_parallel_rank(): return get_state().pp_rank
def get_expert_model_parallel_group(): return get_state().group("ep")
def get_expert_model_parallel_world_size(): return get_state().dims.ep
def get_expert_model_parallel_rank(): return get_state().ep_rank
def get_expert_tensor_parallel_group(): return get_state().group("etp")
def get_expert_tensor_parallel_world_size(): return get_state().dims.etp
def get_expert_data_parallel_group(): return get_state().group("edp")
def get_model_parallel_group(): return get_state().group("mp")
def get_embedding_group(): return get_state().group("embd")
def is_pipeline_first_stage(): return get_state().is_first_stage
def is_pipeline_last_stage(): return get_state().is_last_stage
