"""Mixture-of-experts layer: router, all-to-all token dispatcher over the expert-parallel group,
grouped expert MLP, optional shared expert.

Counterpart of Megatron's ``MoELayer`` / ``TopKRouter`` / ``MoEAlltoAllTokenDispatcher`` /
``TEGroupedMLP`` that the reference wires in its specs
(loongforge/models/foundation/qwen3/qwen_layer_spec.py:30-69,
loongforge/models/foundation/deepseek/deepseek_layer_spec.py:153-205); routing semantics follow the
in-tree copy of the routing function (loongforge/models/foundation/ernie4_5_vl/ernie_router.py:32-140).
Parameter names: ``router.weight``, ``router.expert_bias``, ``experts.linear_fc{1,2}.weight{e}``
(grouped-GEMM naming, configs/models/qwen3/ckpt_convert/qwen3_moe_convert.yaml:47-82),
``shared_experts.linear_fc{1,2}.weight``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as OF
from ..ops import moe_ops
from ..parallel import layers as PL
from ..parallel import mappings as M
from ..parallel import state as ps
from .config import TransformerConfig

# Aux-loss values of the current step, keyed by name; the trainer logs and clears them
# (reference: MoE aux-loss tracker, loongforge/train/training_utils.py:2203-2242).
AUX_LOSS_TRACKER = {}


def track_aux_loss(name: str, value: torch.Tensor, layer: int, num_layers: int):
    t = AUX_LOSS_TRACKER.get(name)
    if t is None or t.numel() < max(num_layers, layer + 1) or t.device != value.device:
        # first use, or a deeper model than the one tracked before (several models in one process)
        old = t
        t = torch.zeros(max(num_layers, layer + 1), dtype=torch.float32, device=value.device)
        if old is not None and old.device == t.device:
            t[:old.numel()] = old
        AUX_LOSS_TRACKER[name] = t
    t[layer] += value.detach().float()


class AuxLossScaler(torch.autograd.Function):
    """Attach an auxiliary loss to an activation: identity forward, and backward adds the aux
    loss's gradient with weight ``scale`` (set to the main loss scale by the trainer)."""

    scale = 1.0

    @staticmethod
    def forward(ctx, x, aux):
        ctx.save_for_backward(aux)
        return x

    @staticmethod
    def backward(ctx, g):
        (aux,) = ctx.saved_tensors
        return g, torch.full_like(aux, AuxLossScaler.scale)


_CURRENT_TOKEN_IDS = {"ids": None}


def set_current_token_ids(ids: Optional[torch.Tensor]) -> None:
    """Token ids of the micro-batch in flight, for hash-routed MoE layers (set by the language model)."""
    _CURRENT_TOKEN_IDS["ids"] = ids


class TopKRouter(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, layer_number: int, device=None):
        super().__init__()
        self.cfg, self.layer_number = cfg, layer_number
        self.moe_index = sum(1 for i in range(layer_number) if cfg.is_moe_layer(i))  # 0-based among MoE layers
        # None: the router sees a sequence shard exactly when sequence parallelism is on; the MoE layer sets True when it
        # shards the tokens over the TP ranks itself (tensor parallelism without sequence parallelism)
        self.tokens_sharded_over_tp: Optional[bool] = None
        E = cfg.num_moe_experts
        w = PL.init_full_then_slice(key + ".weight", (E, cfg.hidden_size), cfg.init_method_std, partition_dim=None,
                                    rank=0, world=1, device=device or "cpu", dtype=torch.float32)
        self.weight = nn.Parameter(w)  # router runs in fp32
        PL.mark_tp(self.weight, None, sequence_parallel=cfg.sequence_parallel)
        if cfg.moe_router_enable_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32, device=device))
            self.register_buffer("local_tokens_per_expert", torch.zeros(E, dtype=torch.float32, device=device),
                                 persistent=False)
        else:
            self.expert_bias = None

    def forward(self, x: torch.Tensor, seq_lens: Optional[List[int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """x [T, H] -> (probs [T, E] fp32 (zero outside the top-k), routing_map [T, E] bool)."""
        cfg = self.cfg
        logits = torch.nn.functional.linear(x.float(), self.weight.float())
        # Under sequence parallelism this rank routes a SHARD of the micro-batch's tokens and the router weight's
        # gradient is summed over the TP ranks afterwards: every rank therefore contributes its share of the
        # whole-micro-batch auxiliary losses (reference: Megatron reduces the aux-loss statistics over the tp-cp group).
        st = ps.get_state()
        sharded = cfg.sequence_parallel if self.tokens_sharded_over_tp is None else self.tokens_sharded_over_tp
        sp_group = st.group("tp") if (sharded and st.dims.tp > 1 and dist.is_initialized()) else None
        sp_n = st.dims.tp if sp_group is not None else 1
        if cfg.moe_z_loss_coeff:
            z = torch.logsumexp(logits, dim=-1).square().mean() * (cfg.moe_z_loss_coeff / sp_n)
            track_aux_loss("z_loss", self._whole(z, sp_group) / cfg.moe_z_loss_coeff, self.layer_number, cfg.num_layers)
            logits = AuxLossScaler.apply(logits, z)
        ids = _CURRENT_TOKEN_IDS["ids"]
        if self.moe_index < cfg.moe_n_hash_layers and ids is not None:
            if sp_n > 1 and ids.numel() == logits.shape[0] * sp_n:  # this rank's sequence shard of the token ids
                ids = ids[st.tp_rank * logits.shape[0]:(st.tp_rank + 1) * logits.shape[0]]
            if ids.numel() != logits.shape[0]:
                raise RuntimeError(f"hash routing got {ids.numel()} token ids for {logits.shape[0]} routed tokens")
            # experts are fixed by the token id; the gate only weights them (scores normalised over the k picks)
            idx = moe_ops.hash_routing(ids, cfg.num_moe_experts, cfg.moe_router_topk)
            s = torch.sqrt(torch.nn.functional.softplus(logits)) if cfg.moe_router_score_function == "sqrtsoftplus" \
                else (torch.sigmoid(logits) if cfg.moe_router_score_function == "sigmoid" else logits.softmax(-1))
            vals = s.gather(1, idx)
            vals = vals / (vals.sum(-1, keepdim=True) + 1e-20) * (cfg.moe_router_topk_scaling_factor or 1.0)
            probs = torch.zeros_like(s).scatter(1, idx, vals)
            routing_map = torch.zeros_like(s, dtype=torch.bool).scatter(1, idx, True)
            return probs, routing_map
        probs, routing_map, scores_for_aux = moe_ops.topk_routing(
            logits, cfg.moe_router_topk, score_function=cfg.moe_router_score_function,
            pre_softmax=cfg.moe_router_pre_softmax, expert_bias=self.expert_bias,
            num_groups=cfg.moe_router_num_groups, group_topk=cfg.moe_router_group_topk,
            scaling_factor=cfg.moe_router_topk_scaling_factor)
        if self.expert_bias is not None and self.training:
            with torch.no_grad():
                self.local_tokens_per_expert += routing_map.sum(0).float()
        if self.training and cfg.moe_aux_loss_coeff and cfg.moe_router_load_balancing_type != "none":
            kind = cfg.moe_router_load_balancing_type
            if kind == "seq_aux_loss" and seq_lens is not None:
                aux = moe_ops.seq_aux_loss(scores_for_aux, routing_map, cfg.moe_router_topk, seq_lens,
                                           cfg.moe_aux_loss_coeff)
            else:
                tpe = routing_map.sum(0)
                if sp_group is not None:
                    # f_e over ALL tokens of the micro-batch, P_e from the local shard: the ranks' losses add up to the
                    # loss of the whole micro-batch (1 / T^2 with the global T)
                    tpe = tpe.float()
                    dist.all_reduce(tpe, group=sp_group)
                aux = moe_ops.switch_aux_loss(scores_for_aux, tpe, cfg.moe_router_topk, cfg.moe_aux_loss_coeff) \
                    / (sp_n * sp_n)
            track_aux_loss("load_balancing_loss", self._whole(aux, sp_group) / cfg.moe_aux_loss_coeff, self.layer_number,
                           cfg.num_layers)
            probs = AuxLossScaler.apply(probs, aux)
        return probs, routing_map

    @staticmethod
    def _whole(value: torch.Tensor, group) -> torch.Tensor:
        """Detached value summed over the sequence-parallel ranks (for logging)."""
        v = value.detach().clone()
        if group is not None:
            dist.all_reduce(v, group=group)
        return v

    @torch.no_grad()
    def update_expert_bias(self, group=None):
        """Aux-loss-free balancing: raise the bias of under-loaded experts, lower over-loaded ones
        (reference call site: loongforge/train/training_utils.py:2203-2226)."""
        if self.expert_bias is None:
            return
        cnt = self.local_tokens_per_expert.clone()
        if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(cnt, group=group)
        self.expert_bias += torch.sign(cnt.mean() - cnt) * self.cfg.moe_router_bias_update_rate
        self.local_tokens_per_expert.zero_()


class GroupedLinear(nn.Module):
    """E_local independent [out, in] weights named ``weight0..weight{E-1}``; applies each to its
    contiguous slice of a token list sorted by expert."""

    def __init__(self, num_local: int, first_global: int, in_f: int, out_f: int, key: str, std: float,
                 cfg: TransformerConfig, device=None, stride: int = 1, etp_dim: Optional[int] = None,
                 etp_rank: int = 0, etp_size: int = 1):
        """``etp_dim``: dimension along which every expert weight is sharded over the expert-tensor-parallel group
        (0 for FC1, column parallel with `stride` blocks; 1 for FC2, row parallel); None = not sharded."""
        super().__init__()
        self.num_local = num_local
        shard = etp_dim if etp_size > 1 else None
        for e in range(num_local):
            w = PL.init_full_then_slice(f"{key}.weight{first_global + e}", (out_f, in_f), std, partition_dim=shard,
                                        rank=etp_rank if shard is not None else 0,
                                        world=etp_size if shard is not None else 1, device=device or "cpu",
                                        dtype=cfg.params_dtype, stride=stride if shard == 0 else 1)
            p = nn.Parameter(w)
            PL.mark_tp(p, shard, stride=stride if shard == 0 else 1)
            p.is_expert = True
            p.partition_stride = stride
            p.expert_global_index = first_global + e  # checkpoints name experts by their global index
            self.register_parameter(f"weight{e}", p)

    def weights(self):
        return [getattr(self, f"weight{e}") for e in range(self.num_local)]

    def forward(self, x: torch.Tensor, tokens_per_expert: List[int]) -> torch.Tensor:
        return moe_ops.grouped_linear(x, self.weights(), tokens_per_expert)


class GroupedMLP(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, num_local: int, first_global: int, device=None,
                 etp_rank: int = 0, etp_size: int = 1):
        super().__init__()
        f = cfg.moe_ffn_hidden_size
        glu = cfg.gated_linear_unit
        assert f % etp_size == 0, "moe_ffn_hidden_size must divide by the expert tensor parallel size"
        etp = dict(etp_rank=etp_rank, etp_size=etp_size)
        self.linear_fc1 = GroupedLinear(num_local, first_global, cfg.hidden_size, f * (2 if glu else 1),
                                        key + ".linear_fc1", cfg.init_method_std, cfg, device, stride=2 if glu else 1,
                                        etp_dim=0, **etp)
        self.linear_fc2 = GroupedLinear(num_local, first_global, f, cfg.hidden_size, key + ".linear_fc2",
                                        cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers), cfg, device,
                                        etp_dim=1, **etp)
        self.glu = glu
        self.act = cfg.activation
        self.swiglu_limit = cfg.swiglu_limit

    def forward(self, x, tokens_per_expert, row_probs=None):
        """``row_probs`` [rows]: router probability of each received row, multiplied in before FC2
        (dispatchers that sum expert outputs unweighted pass it; Megatron's weighted-SwiGLU form)."""
        h = self.linear_fc1(x, tokens_per_expert)
        if self.glu and self.act == "swiglu" and self.swiglu_limit:
            from .transformer import clamped_swiglu
            h = clamped_swiglu(h, self.swiglu_limit)
        elif self.glu and self.act == "swiglu":
            h = OF.swiglu(h)
        elif self.glu:
            g, u = h.chunk(2, -1)
            h = torch.nn.functional.gelu(g) * u
        else:
            h = torch.nn.functional.gelu(h)
        if row_probs is not None:
            h = h * row_probs.unsqueeze(-1).to(h.dtype)
        return self.linear_fc2(h, tokens_per_expert)


class AlltoAllDispatcher:
    """permute -> all-to-all(v) over EP -> sort by local expert; and the exact inverse.
    Splits are exchanged on the host (one small all_to_all of counts), as Megatron's
    alltoall dispatcher does."""

    def __init__(self, num_experts: int, state_name=None):
        st = ps.get_state(state_name)
        self.ep, self.ep_rank, self.group = st.dims.ep, st.ep_rank, st.group("ep")
        self.E = num_experts
        self.E_local = num_experts // self.ep

    def dispatch(self, x, probs, routing_map):
        T, H = x.shape
        # (expert, token) pairs in expert-major order
        emap = routing_map.t().contiguous()
        expert_idx, token_idx = emap.nonzero(as_tuple=True)
        self.token_idx = token_idx
        self.sel_probs = probs.t()[expert_idx, token_idx]
        self.T = T
        permuted = x.index_select(0, token_idx)
        counts = emap.sum(1)  # tokens per global expert (local tokens)
        if self.ep == 1:
            self.tpe = counts.tolist()
            return permuted, self.tpe
        # counts matrix: what every EP rank sends to each of my local experts
        send_counts = counts.view(self.ep, self.E_local)
        recv_counts = torch.empty_like(send_counts)
        if send_counts.is_cuda:
            dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        else:
            M.all_to_all_single(recv_counts, send_counts.contiguous(), None, None, self.group)
        self.in_splits = send_counts.sum(1).tolist()
        rc = recv_counts.cpu()
        self.out_splits = rc.sum(1).tolist()
        recv = M.all_to_all(permuted, self.group, self.out_splits, self.in_splits)
        # received order is [src rank][local expert]; experts need [local expert][src rank]
        chunk_sizes = rc.reshape(-1).tolist()
        order = [s * self.E_local + e for e in range(self.E_local) for s in range(self.ep)]
        self.chunk_sizes, self.order = chunk_sizes, order
        chunks = recv.split(chunk_sizes, 0)
        sorted_tokens = torch.cat([chunks[i] for i in order], 0) if len(chunks) > 1 else recv
        self.tpe = rc.sum(0).tolist()
        return sorted_tokens, self.tpe

    def combine(self, y, sel_probs=None):
        """`sel_probs`: the probabilities `dispatch` left in ``self.sel_probs`` (passed explicitly by callers that cut
        the autograd graph between the two calls)."""
        sel_probs = self.sel_probs if sel_probs is None else sel_probs
        if self.ep > 1:
            sizes_sorted = [self.chunk_sizes[i] for i in self.order]
            chunks = y.split(sizes_sorted, 0)
            inv = [0] * len(self.order)
            for pos, i in enumerate(self.order):
                inv[i] = pos
            y = torch.cat([chunks[inv[i]] for i in range(len(self.order))], 0) if len(chunks) > 1 else y
            y = M.all_to_all(y, self.group, self.in_splits, self.out_splits)
        y = y * sel_probs.to(y.dtype).unsqueeze(-1)
        out = torch.zeros(self.T, y.shape[1], dtype=y.dtype, device=y.device)
        return out.index_add(0, self.token_idx, y)


class MoELayer(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, layer_number: int, *, device=None, parallel_state=None):
        super().__init__()
        self.cfg, self.layer_number, self.state_name = cfg, layer_number, parallel_state
        st = ps.get_state(parallel_state)
        E, ep = cfg.num_moe_experts, st.dims.ep
        assert E % ep == 0, "num_moe_experts must divide by expert parallel size"
        self.E_local = E // ep
        self.router = TopKRouter(cfg, key + ".router", layer_number, device=device)
        if st.dims.tp > 1:
            # the router always sees a token shard under TP (see forward): its gradient is a partial sum on every rank
            self.router.weight.tp_partial_grad = True
        self.etp = st.dims.etp
        self.experts = GroupedMLP(cfg, key + ".experts", self.E_local, st.ep_rank * self.E_local, device=device,
                                  etp_rank=st.etp_rank, etp_size=st.dims.etp)
        if cfg.moe_shared_expert_intermediate_size:
            from .transformer import MLP
            self.shared_experts = MLP(cfg, key + ".shared_experts", ffn_hidden=cfg.moe_shared_expert_intermediate_size,
                                      fused_norm=False, device=device, parallel_state=parallel_state,
                                      sequence_parallel=False)
            if cfg.moe_shared_expert_gate:
                # y_shared * sigmoid(x . g): one gate logit per token (Qwen2-MoE / Qwen3-Next / Qwen3.5; stored as
                # mlp.shared_experts.gate_weight, configs/models/qwen3_next/ckpt_convert/qwen3_next_moe_convert.yaml:132-134)
                w = PL.init_full_then_slice(key + ".shared_experts.gate_weight", (1, cfg.hidden_size),
                                            cfg.init_method_std, partition_dim=None, rank=0, world=1,
                                            device=device or "cpu", dtype=cfg.params_dtype)
                self.shared_experts.gate_weight = nn.Parameter(w)
                # applied to this rank's token shard under sequence parallelism: partial gradient there
                PL.mark_tp(self.shared_experts.gate_weight, None, sequence_parallel=cfg.sequence_parallel)
        else:
            self.shared_experts = None
        self.dispatcher = AlltoAllDispatcher(E, parallel_state)
        self.peer_dispatcher = None
        if cfg.moe_token_dispatcher_type == "peer":
            from ..parallel.moe_peer import PeerDispatcher
            self.peer_dispatcher = PeerDispatcher(E, cfg.hidden_size, ep, st.ep_rank, st.group("ep") if ep > 1 else None,
                                                  cfg.moe_peer_capacity_factor)

    # The layer is five stages with explicit tensor interfaces: route (compute) -> dispatch_tokens (communication)
    # -> run_experts (compute) -> combine_tokens (communication) -> finish (compute). ``forward`` runs them back to
    # back; the all-to-all overlap schedule (runtime/a2a_overlap.py) runs the same five methods as separate autograd
    # segments so that one micro-batch's exchange sits under another's compute (reference:
    # loongforge/models/omni_models/model_chunk_schedule_plan.py:203-305, node split
    # loongforge/models/omni_models/fine_grained_callables.py:704-1060).

    def route(self, x: torch.Tensor, seq_lens=None):
        """-> (x_loc, probs, routing_map): the tokens this rank routes, their probabilities [T, E] and the map.
        Experts are replicated over the TP ranks (or sliced over them, ETP) and their gradients are summed over those
        ranks, so every rank must route a DIFFERENT part of the tokens. Sequence parallelism delivers shards already;
        without it the layer shards its input here and gathers its output."""
        st = ps.get_state(self.state_name)
        if st.dims.tp > 1 and not self.cfg.sequence_parallel:
            self.router.tokens_sharded_over_tp = True
            x = M.scatter_to_sequence_parallel_region(x, st.group("tp"))
        probs, routing_map = self.router(x, seq_lens)
        return x, probs, routing_map

    def _use_peer(self, x) -> bool:
        return self.etp == 1 and self.peer_dispatcher is not None and x.is_cuda and x.dtype == torch.bfloat16

    def dispatch_tokens(self, x_loc, probs, routing_map):
        """-> (tokens sorted by local expert, aux, tokens_per_expert). `aux` are the probabilities the later stages
        need: per received row with the peer dispatcher (applied on the expert side), per sent (token, expert) pair
        with the all-to-all dispatcher (applied in the combine)."""
        if self.etp > 1:
            # Expert tensor parallelism: the ranks of an ETP group hold slices of every expert's FFN width. They first
            # share their tokens (all-gather) and run the same dispatch. Each rank back-propagates only through ITS
            # slices of the expert weights, so the gradients of the gathered tokens and probabilities are partial
            # sums: reduce-scatter them in backward.
            g = ps.get_state(self.state_name).group("etp")
            x_loc = M.gather_from_sequence_parallel_region(x_loc, g, True)
            probs = M.gather_from_sequence_parallel_region(probs, g, True)
            routing_map = M.gather_from_sequence_parallel_region(routing_map.to(torch.uint8), g, False).bool()
        if self._use_peer(x_loc):
            # indices of the k selected experts of every token (order within a token is irrelevant)
            topk_idx = routing_map.to(torch.float16).topk(self.cfg.moe_router_topk, dim=1).indices
            tokens, tpe, row_probs = self.peer_dispatcher.dispatch(x_loc, probs, topk_idx)
            return tokens, row_probs, tpe
        tokens, tpe = self.dispatcher.dispatch(x_loc, probs, routing_map)
        return tokens, self.dispatcher.sel_probs, tpe

    def run_experts(self, tokens, aux, tpe, x_loc, x_full):
        """-> (y, y_shared or None). The shared expert belongs to this compute stage: it only needs the layer input,
        so in the overlap schedule it also covers the exchange of the routed tokens."""
        y = self.experts(tokens, tpe, aux) if self._use_peer(x_loc) else self.experts(tokens, tpe)
        ys = None
        if self.shared_experts is not None:
            st = ps.get_state(self.state_name)
            if st.dims.tp > 1:
                # shared expert is tensor parallel over the full token set of the TP group
                g = st.group("tp")
                xs = M.gather_from_sequence_parallel_region(x_loc, g, False) if self.cfg.sequence_parallel else x_full
                ys = self.shared_experts(xs)
                if self.cfg.sequence_parallel:
                    ys = M.scatter_to_sequence_parallel_region(ys, g)
            else:
                ys = self.shared_experts(x_loc)
        return y, ys

    def combine_tokens(self, y, aux, x_loc):
        if self._use_peer(x_loc):
            return self.peer_dispatcher.combine(y)
        out = self.dispatcher.combine(y, aux)
        if self.etp > 1:
            # partial FC2 sums of the slices: reduce-scatter back to each rank's own tokens
            out = M.reduce_scatter_to_sequence_parallel_region(out, ps.get_state(self.state_name).group("etp"))
        return out

    def finish(self, out, ys, x_loc, x_full):
        st = ps.get_state(self.state_name)
        local_shard = st.dims.tp > 1 and not self.cfg.sequence_parallel
        if local_shard:
            out = M.gather_from_sequence_parallel_region(out, st.group("tp"), False)
        if ys is not None:
            # the tokens that `out` holds on this rank
            x_out = x_loc if (st.dims.tp > 1 and self.cfg.sequence_parallel) or st.dims.tp == 1 else x_full
            gate_w = getattr(self.shared_experts, "gate_weight", None)
            if gate_w is not None:
                ys = ys * torch.sigmoid(torch.nn.functional.linear(x_out, gate_w).float()).to(ys.dtype)
            out = out + ys
        return out

    def forward(self, x: torch.Tensor, seq_lens=None) -> torch.Tensor:
        x_loc, probs, routing_map = self.route(x, seq_lens)
        tokens, aux, tpe = self.dispatch_tokens(x_loc, probs, routing_map)
        y, ys = self.run_experts(tokens, aux, tpe, x_loc, x)
        out = self.combine_tokens(y, aux, x_loc)
        return self.finish(out, ys, x_loc, x)
