"""Full heterogeneous data parallelism for the vision encoder: while the language model is sharded over a
model-parallel group (TP x PP x CP ranks that all see the SAME micro-batches), the encoder is small and replicated, so
the ranks of that group each encode a DIFFERENT subset of the step's micro-batches — all encoder rounds run before the
pipeline starts — and exchange the resulting embeddings; after the pipeline's backward the embedding gradients travel
back to the rank that encoded them, which then runs the encoder backward (reference:
loongforge/train/training_utils.py:1484-1560 full-hetero path, loongforge/train/initialize.py:251-280 micro-batch
arithmetic, omni_combination_model.py:461-579; embeddings may be parked in host memory, runtime/offload.py).

Usage per step::

    runner = FullHeteroEncoderRunner(group, encode_fn)
    embs = runner.encode_all(inputs_per_microbatch)      # list over micro-batches, identical on every rank
    ... pipeline forward / backward using embs[i] (leaf tensors that collect .grad on the ranks that use them) ...
    runner.backward(contributes=is_first_stage_and_tp_rank0)   # gradients to owners, encoder backward
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def owner_of(microbatch: int, group_size: int) -> int:
    return microbatch % group_size


def rounds(num_microbatches: int, group_size: int) -> int:
    """Encoder forward rounds every rank runs (the last round may be idle on some ranks)."""
    return (num_microbatches + group_size - 1) // group_size


class FullHeteroEncoderRunner:
    def __init__(self, group, encode_fn: Callable[[object], torch.Tensor], offloader=None):
        self.group, self.encode_fn, self.offloader = group, encode_fn, offloader
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.ranks = dist.get_process_group_ranks(group) if self.world > 1 else [0]
        self._own: dict = {}      # microbatch -> embedding with autograd graph (owner only)
        self._leaves: List[torch.Tensor] = []
        self._parked: dict = {}    # microbatch -> host handle of an offloaded embedding

    def encode_all(self, inputs: Sequence[object]) -> List[torch.Tensor]:
        self._own.clear()
        self._leaves = []
        n = len(inputs)
        for i in range(n):
            if owner_of(i, self.world) == self.rank:
                self._own[i] = self.encode_fn(inputs[i])
        for i in range(n):
            o = owner_of(i, self.world)
            if self.world == 1:
                leaf = self._own[i].detach().clone().requires_grad_(True)
            else:
                src = self.ranks[o]
                mine = self._own.get(i)
                dev = mine.device if mine is not None else self._device_hint(inputs)
                meta = torch.zeros(3, dtype=torch.long, device=dev)
                if mine is not None:
                    meta[0], meta[1] = mine.shape[0], mine.shape[1]
                    meta[2] = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[mine.dtype]
                dist.broadcast(meta, src, group=self.group)
                rows, cols, code = meta.tolist()
                dtype = [torch.float32, torch.bfloat16, torch.float16][code]
                buf = mine.detach().clone() if mine is not None else torch.empty(rows, cols, dtype=dtype, device=dev)
                dist.broadcast(buf, src, group=self.group)
                leaf = buf.requires_grad_(True)
            if self.offloader is not None:
                # park the embedding in pinned host memory until its micro-batch enters the pipeline (`leaf(i)`)
                self._parked[i] = self.offloader.offload(leaf.detach())
                leaf = None
            self._leaves.append(leaf)
        return self._leaves

    def leaf(self, i: int) -> torch.Tensor:
        """The embedding of micro-batch i as a leaf tensor that collects ``.grad``; brings it back from host memory
        first when an offloader is in use."""
        if self._leaves[i] is None:
            self._leaves[i] = self.offloader.reload(self._parked.pop(i)).detach().clone().requires_grad_(True)
        return self._leaves[i]

    @staticmethod
    def _device_hint(inputs):
        for x in inputs:
            if torch.is_tensor(x):
                return x.device
            if isinstance(x, (tuple, list)) and x and torch.is_tensor(x[0]):
                return x[0].device
        return torch.device("cpu")

    def backward(self, contributes: bool = True) -> None:
        """Every rank calls this once after the pipeline backward. Ranks with ``contributes=False`` (replicas that hold a
        duplicate of the same gradient, or stages that never used the embeddings) send zeros."""
        for i in range(len(self._leaves)):
            leaf = self.leaf(i)
            g = leaf.grad if (contributes and leaf.grad is not None) else torch.zeros_like(leaf)
            if self.world > 1:
                g = g.contiguous()
                dist.reduce(g, self.ranks[owner_of(i, self.world)], op=dist.ReduceOp.SUM, group=self.group)
            if i in self._own:
                self._own[i].backward(g.to(self._own[i].dtype))
        self._own.clear()
        self._leaves = []
