"""LoRA adapters for the tensor-parallel linears (loongforge/models/common/peft/lora.py:58-346,
lora_layers.py:37-710, utils.py:60-118).

* ``apply_lora(model, rank, alpha, targets)`` freezes the base weights and wraps every linear
  whose name ends with a target (``linear_qkv``, ``linear_proj``, ``linear_fc1``, ``linear_fc2``)
  with trainable ``lora_A`` / ``lora_B``. For column-parallel layers A is replicated and B is
  sharded on the output; for row-parallel layers A is sharded on the input and B replicated, so
  the low-rank path needs no extra collective beyond the wrapped layer's own.
* ``canonical=True`` gives the packed QKV and the gate/up projections one adapter pair per logical
  matrix (q, k, v / gate, up) as the reference's canonical LoRA does.
* ``merge_lora`` folds ``B @ A * alpha/rank`` into the base weights; ``adapter_state_dict`` keeps only
  adapter tensors (adapter-only checkpoints).
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from ..ops import functional as OF
from ..parallel import layers as PL
from ..parallel import mappings as M
from ..parallel import state as ps


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Module, rank: int, alpha: float, dropout: float = 0.0, key: str = "lora",
                 splits: Optional[List[int]] = None):
        super().__init__()
        self.base = base
        self.rank, self.scale = rank, alpha / rank
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        w = base.weight
        out_local, in_local = w.shape
        dev, dt = w.device, w.dtype
        self.is_row = isinstance(base, PL.RowParallelLinear)
        # splits: output row counts of the logical matrices inside a fused weight (canonical LoRA)
        self.splits = splits or [out_local]
        n = len(self.splits)
        tp, tp_rank = getattr(base, "tp", 1) or 1, getattr(base, "tp_rank", 0)
        in_full = in_local * tp if self.is_row else in_local
        # A is drawn for the FULL input width from a seed that depends only on the layer's layout-independent name, then
        # sliced: the adapters (and the run) do not depend on the TP / PP layout. Variance 1 / (3 fan_in), that of the
        # usual Kaiming-uniform adapter init.
        a = PL.init_full_then_slice(getattr(base, "init_key", key) + ".lora_A", (n * rank, in_full),
                                    1.0 / math.sqrt(3.0 * in_full), partition_dim=1 if self.is_row else None,
                                    rank=tp_rank, world=tp, device=dev, dtype=dt)
        self.lora_A = nn.Parameter(a)
        self.lora_B = nn.Parameter(torch.zeros(out_local, rank, dtype=dt, device=dev))
        PL.mark_tp(self.lora_A, 1 if self.is_row else None, shards=tp, shard_rank=tp_rank)
        PL.mark_tp(self.lora_B, None if self.is_row else 0, shards=tp, shard_rank=tp_rank)
        if tp > 1:
            # the replicated factor sits next to a sharded one, so each rank computes only a partial gradient for it
            # (column parallel: A sees the gradient of the local output slice; row parallel: B sees the local partial
            # sum of A's output): summed over the TP group by the trainer
            (self.lora_B if self.is_row else self.lora_A).tp_partial_grad = True
        for p in base.parameters():
            p.requires_grad_(False)

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    # callers that fuse neighbouring ops into a plain linear check `tp == 1`; an adapted layer opts out
    tp = 0

    def _delta(self, x):
        """Low-rank path on the tensor the base GEMM sees (after all-gather / before reduction)."""
        h = OF.linear(self.dropout(x), self.lora_A)  # [T, n*rank]
        outs, r0, o0 = [], 0, 0
        for rows in self.splits:
            outs.append(OF.linear(h[..., r0:r0 + self.rank], self.lora_B[o0:o0 + rows]))
            r0 += self.rank
            o0 += rows
        return (outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)) * self.scale

    def forward(self, x, residual=None):
        base = self.base
        st = ps.get_state(base.state_name)
        g = st.group(base.group_kind)
        if self.is_row:
            y = base(x, residual)
            d = self._delta(x)
            if base.tp > 1:
                d = (M.reduce_scatter_to_sequence_parallel_region(d, g) if base.sequence_parallel
                     else M.reduce_from_tensor_model_parallel_region(d, g))
            return y + d
        y = base(x)
        xin = x
        norm = getattr(base, "_norm", None)
        if norm is not None:  # fused norm + linear: the adapter sees the normalised input too
            from .transformer import apply_norm
            xin = apply_norm(x, base.layer_norm_weight, base.layer_norm_bias, *norm)
        if base.tp > 1:
            xin = (M.gather_from_sequence_parallel_region(xin, g, True) if base.sequence_parallel
                   else M.copy_to_tensor_model_parallel_region(xin, g))
        return y + self._delta(xin)

    @torch.no_grad()
    def merged_delta(self) -> torch.Tensor:
        outs, r0, o0 = [], 0, 0
        for rows in self.splits:
            outs.append(self.lora_B[o0:o0 + rows].float() @ self.lora_A[r0:r0 + self.rank].float())
            r0 += self.rank
            o0 += rows
        return torch.cat(outs, 0) * self.scale


def _canonical_splits(name: str, mod) -> Optional[List[int]]:
    out_local = mod.weight.shape[0]
    if name.endswith("linear_fc1") and getattr(mod.weight, "partition_stride", 1) == 2:
        return [out_local // 2, out_local // 2]
    return None


def apply_lora(model: nn.Module, rank: int = 16, alpha: float = 32, dropout: float = 0.0,
               targets: Iterable[str] = ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"),
               canonical: bool = False, freeze_rest: bool = True) -> List[str]:
    """Wrap target linears in place; returns the wrapped module names. Everything else is frozen (``freeze_rest``)."""
    targets = tuple(targets)
    if freeze_rest:
        for p in model.parameters():
            p.requires_grad_(False)
    wrapped = []
    for name, mod in list(model.named_modules()):
        if not isinstance(mod, (PL.ColumnParallelLinear, PL.RowParallelLinear)):
            continue
        if not name.split(".")[-1] in targets:
            continue
        parent = model.get_submodule(".".join(name.split(".")[:-1])) if "." in name else model
        splits = _canonical_splits(name, mod) if canonical else None
        setattr(parent, name.split(".")[-1], LoRALinear(mod, rank, alpha, dropout, key=name, splits=splits))
        wrapped.append(name)
    return wrapped


VLM_COMPONENTS = ("foundation", "image_encoder", "image_projector")


def apply_vlm_lora(omni: nn.Module, *, apply_to_foundation: bool = True, apply_to_image_encoder: bool = False,
                   apply_to_image_projector: bool = False, frozen: Iterable[str] = (), **lora_kw) -> Dict[str, List[str]]:
    """Adapters per component of a vision-language model (reference: the component prefixes of
    loongforge/train/training_utils.py:645-700). A component that gets adapters has its base weights frozen and its
    adapters trained; a component without adapters keeps its own training state (trainable, or frozen when it is listed
    in `frozen`). Asking for adapters on a component that is also listed as frozen is an error, as in the reference."""
    want = {"foundation": apply_to_foundation, "image_encoder": apply_to_image_encoder,
            "image_projector": apply_to_image_projector}
    frozen = set(frozen)
    for comp in VLM_COMPONENTS:
        if want[comp] and comp in frozen:
            raise ValueError(f"cannot freeze the {comp.replace('_', ' ')} when adapters are applied to it")
    enc = getattr(omni, "encoder_model", None)
    mods = {"foundation": getattr(omni, "foundation_model", None),
            "image_encoder": getattr(enc, "image_encoder", None) if enc is not None else None,
            "image_projector": getattr(enc, "image_projector", None) if enc is not None else None}
    wrapped: Dict[str, List[str]] = {}
    for comp in VLM_COMPONENTS:
        m = mods[comp]
        if m is None:
            continue
        if want[comp]:
            wrapped[comp] = apply_lora(m, **lora_kw)
        elif comp in frozen:
            for p in m.parameters():
                p.requires_grad_(False)
    return wrapped


@torch.no_grad()
def merge_lora(model: nn.Module) -> int:
    """Fold every adapter into its base weight and unwrap; returns the number of merged layers."""
    n = 0
    for name, mod in list(model.named_modules()):
        if isinstance(mod, LoRALinear):
            mod.base.weight.add_(mod.merged_delta().to(mod.base.weight.dtype))
            for p in mod.base.parameters():
                p.requires_grad_(True)
            parent = model.get_submodule(".".join(name.split(".")[:-1])) if "." in name else model
            setattr(parent, name.split(".")[-1], mod.base)
            n += 1
    return n


def adapter_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v for k, v in model.state_dict().items() if ".lora_A" in k or ".lora_B" in k}
