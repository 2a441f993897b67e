"""Tensor-parallel building blocks: column/row-parallel linears (with Megatron sequence
parallelism), vocabulary-parallel embedding.

Replaces what the reference takes from Megatron-Core / TransformerEngine
(`TELayerNormColumnParallelLinear`, `TERowParallelLinear`, `VocabParallelEmbedding`; selected in
loongforge/models/dispatch.py:45-54 and used by the layer specs, e.g.
loongforge/models/foundation/llama/llama_layer_spec.py:37-75).

Weight layout is Megatron's: ``[out, in]`` with column-parallel sharding on dim 0 and
row-parallel on dim 1, so checkpoints interchange. Initialisation draws the FULL tensor from a
generator keyed by the parameter's global name and slices the local shard, which makes the
initial model independent of the parallel layout.
"""
from __future__ import annotations

import zlib
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as OF
from . import mappings as M
from . import state as ps

_INIT_SEED = {"seed": 1234}


def set_init_seed(seed: int) -> None:
    _INIT_SEED["seed"] = int(seed)


def init_full_then_slice(key: str, full_shape, std: float, *, partition_dim: Optional[int], rank: int, world: int,
                         device, dtype, mean: float = 0.0, stride: int = 1) -> torch.Tensor:
    """N(mean, std) draw of the full tensor (deterministic in `key`), sliced for (rank, world).

    ``stride`` > 1 handles fused tensors such as SwiGLU FC1 = [gate; up]: each of the `stride`
    row blocks is sharded separately and the local pieces concatenated, which is the layout
    of the reference's converters (tools/convert_checkpoint/mcore/mcore_base.py:375-377,422-423).
    """
    g = torch.Generator(device="cpu")
    g.manual_seed((zlib.crc32(key.encode()) + _INIT_SEED["seed"]) & 0x7FFFFFFF)
    dev = torch.device(device)
    numel = 1
    for s in full_shape:
        numel *= s
    if dev.type == "cuda" and numel > (1 << 22):
        gg = torch.Generator(device=dev)
        gg.manual_seed((zlib.crc32(key.encode()) + _INIT_SEED["seed"]) & 0x7FFFFFFF)
        full = torch.empty(full_shape, dtype=torch.float32, device=dev).normal_(mean, std, generator=gg)
    else:
        full = torch.empty(full_shape, dtype=torch.float32).normal_(mean, std, generator=g).to(dev)
    if partition_dim is None or world == 1:
        return full.to(dtype)
    if stride == 1:
        return full.chunk(world, dim=partition_dim)[rank].contiguous().to(dtype)
    blocks = full.chunk(stride, dim=partition_dim)
    return torch.cat([b.chunk(world, dim=partition_dim)[rank] for b in blocks], dim=partition_dim).contiguous().to(dtype)


def mark_tp(param: torch.Tensor, partition_dim: Optional[int], stride: int = 1, sequence_parallel: bool = False,
            shards: Optional[int] = None, shard_rank: int = 0):
    """Attributes consumed by checkpointing, grad-norm and the SP gradient all-reduce.

    ``shards`` / ``shard_rank``: tensor-parallel size and rank of the parallel state the OWNING module was built for.
    A module of a state with a smaller TP degree than the job's main state (a vision encoder with TP 1 beside a
    decoder with TP 2) is replicated over the main TP group: checkpoints then write it once with its own sharding,
    and the gradient norm counts it once."""
    param.tensor_model_parallel = partition_dim is not None
    if shards is not None:
        param.tp_shards, param.tp_shard_rank = shards, shard_rank
    param.partition_dim = -1 if partition_dim is None else partition_dim
    param.partition_stride = stride
    param.sequence_parallel = sequence_parallel
    return param


def mark_tp_partial_grad(module: nn.Module) -> None:
    """Parameters of `module` are replicated over the TP group but applied to THIS rank's heads only, so each rank
    holds a partial gradient that the trainer sums over the TP group."""
    for p in module.parameters():
        p.tp_partial_grad = True


def _linear(module, x, weight, bias=None, residual=None):
    """The module's GEMM in the precision chosen for it (``module.gemm_precision``: unset / 'bf16' -> parameter dtype,
    'fp8' -> block-quantised e4m3 forward and input-gradient GEMMs)."""
    if getattr(module, "gemm_precision", None) == "fp8":
        from ..ops import quant
        return quant.fp8_linear(x, weight, bias, residual)
    return OF.linear(x, weight, bias, residual)


class ColumnParallelLinear(nn.Module):
    """Y = X W^T with W sharded on the output dim. With sequence parallelism the input is
    ``[T/tp, in]`` and is all-gathered along tokens first (backward: reduce-scatter of dX)."""

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False, gather_output: bool = False,
                 init_std: float = 0.02, key: str = "col", sequence_parallel: bool = False, stride: int = 1,
                 params_dtype=torch.float32, device=None, parallel_state: Optional[str] = None,
                 tp_comm_overlap: bool = False, is_expert: bool = False):
        super().__init__()
        st = ps.get_state(parallel_state)
        self.state_name = parallel_state
        self.init_key = key  # layout-independent name of this layer (global layer index), also seeds adapters
        self.tp = st.dims.etp if is_expert else st.dims.tp
        self.tp_rank = st.etp_rank if is_expert else st.tp_rank
        self.group_kind = "etp" if is_expert else "tp"
        assert out_features % (self.tp * stride) == 0, f"{key}: out_features {out_features} not divisible by tp"
        self.in_features, self.out_features = in_features, out_features
        self.out_local = out_features // self.tp
        self.gather_output = gather_output
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.tp_comm_overlap = tp_comm_overlap and self.tp > 1
        device = device if device is not None else "cpu"
        w = init_full_then_slice(key + ".weight", (out_features, in_features), init_std, partition_dim=0,
                                 rank=self.tp_rank, world=self.tp, device=device, dtype=params_dtype, stride=stride)
        self.weight = nn.Parameter(w)
        mark_tp(self.weight, 0, stride, shards=self.tp, shard_rank=self.tp_rank)
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.out_local, dtype=params_dtype, device=device))
            mark_tp(self.bias, 0, stride, shards=self.tp, shard_rank=self.tp_rank)
        else:
            self.register_parameter("bias", None)

    def _group(self):
        return ps.get_state(self.state_name).group(self.group_kind)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g = self._group()
        if self.tp > 1:
            if self.sequence_parallel:
                if self.tp_comm_overlap and x.is_cuda:
                    from . import fused_tp
                    y = fused_tp.all_gather_linear(x, self.weight, self.bias, self.state_name)
                    return y
                x = M.gather_from_sequence_parallel_region(x, g, True)
            else:
                x = M.copy_to_tensor_model_parallel_region(x, g)
        y = _linear(self, x, self.weight, self.bias)
        if self.gather_output and self.tp > 1:
            y = M.gather_from_tensor_model_parallel_region(y, g)
        return y


class RowParallelLinear(nn.Module):
    """Y = X W^T with W sharded on the input dim; partial sums are reduce-scattered along
    tokens (sequence parallel) or all-reduced. The bias is added after the reduction."""

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False, input_is_parallel: bool = True,
                 init_std: float = 0.02, key: str = "row", sequence_parallel: bool = False,
                 params_dtype=torch.float32, device=None, parallel_state: Optional[str] = None,
                 tp_comm_overlap: bool = False, is_expert: bool = False):
        super().__init__()
        st = ps.get_state(parallel_state)
        self.state_name = parallel_state
        self.init_key = key  # layout-independent name of this layer (global layer index), also seeds adapters
        self.tp = st.dims.etp if is_expert else st.dims.tp
        self.tp_rank = st.etp_rank if is_expert else st.tp_rank
        self.group_kind = "etp" if is_expert else "tp"
        assert in_features % self.tp == 0
        self.in_features, self.out_features = in_features, out_features
        self.in_local = in_features // self.tp
        self.input_is_parallel = input_is_parallel
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.tp_comm_overlap = tp_comm_overlap and self.tp > 1
        device = device if device is not None else "cpu"
        w = init_full_then_slice(key + ".weight", (out_features, in_features), init_std, partition_dim=1,
                                 rank=self.tp_rank, world=self.tp, device=device, dtype=params_dtype)
        self.weight = nn.Parameter(w)
        mark_tp(self.weight, 1, shards=self.tp, shard_rank=self.tp_rank)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=params_dtype, device=device))
            mark_tp(self.bias, None, sequence_parallel=self.sequence_parallel)
        else:
            self.register_parameter("bias", None)

    def _group(self):
        return ps.get_state(self.state_name).group(self.group_kind)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns ``X W^T (+bias) (+residual)``; `residual` has the OUTPUT's (possibly
        sequence-sharded) shape and is folded into the GEMM / reduction epilogue."""
        g = self._group()
        if self.tp > 1 and not self.input_is_parallel:
            x = M.scatter_to_tensor_model_parallel_region(x, g)
        if self.tp == 1:
            return _linear(self, x, self.weight, self.bias, residual)
        if self.sequence_parallel and self.tp_comm_overlap and x.is_cuda and self.bias is None:
            from . import fused_tp
            return fused_tp.linear_reduce_scatter(x, self.weight, residual, self.state_name)
        y = _linear(self, x, self.weight)
        if self.sequence_parallel:
            y = M.reduce_scatter_to_sequence_parallel_region(y, g)
        else:
            y = M.reduce_from_tensor_model_parallel_region(y, g)
        if self.bias is not None:
            y = y + self.bias
        if residual is not None:
            y = y + residual
        return y


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded on the vocabulary; out-of-shard ids contribute zeros and the
    partial results are summed over TP (reduce-scattered along tokens under SP)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, init_std: float = 0.02,
                 key: str = "embedding.word_embeddings", sequence_parallel: bool = False,
                 params_dtype=torch.float32, device=None, parallel_state: Optional[str] = None):
        super().__init__()
        st = ps.get_state(parallel_state)
        self.state_name = parallel_state
        self.init_key = key  # layout-independent name of this layer (global layer index), also seeds adapters
        self.tp, self.tp_rank = st.dims.tp, st.tp_rank
        assert num_embeddings % self.tp == 0
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.per = num_embeddings // self.tp
        self.vocab_start = self.tp_rank * self.per
        self.vocab_end = self.vocab_start + self.per
        self.sequence_parallel = sequence_parallel and self.tp > 1
        device = device if device is not None else "cpu"
        w = init_full_then_slice(key + ".weight", (num_embeddings, embedding_dim), init_std, partition_dim=0,
                                 rank=self.tp_rank, world=self.tp, device=device, dtype=params_dtype)
        self.weight = nn.Parameter(w)
        mark_tp(self.weight, 0, shards=self.tp, shard_rank=self.tp_rank)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        g = ps.get_state(self.state_name).group("tp")
        if self.tp == 1:
            return torch.nn.functional.embedding(ids, self.weight)
        mask = (ids < self.vocab_start) | (ids >= self.vocab_end)
        local = (ids - self.vocab_start).masked_fill(mask, 0)
        out = torch.nn.functional.embedding(local, self.weight)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        if self.sequence_parallel:
            return M.reduce_scatter_to_sequence_parallel_region(out, g)
        return M.reduce_from_tensor_model_parallel_region(out, g)
