"""Loss reductions (loongforge/train/get_loss_func.py:16-176, loongforge/train/pretrain/pretrain_llm.py:79-132).

``masked_sum_loss`` is the default: sum(loss * mask) with the token count, either normalised per
micro-batch (Megatron default) or left as (sum, count) for per-token normalisation over the global
batch (``--calculate-per-token-loss``). ``loss_weight`` re-weights tokens (e.g. per-sample weights).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

IGNORE_INDEX = -100


def labels_to_mask(labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> Tuple[torch.Tensor, torch.Tensor]:
    mask = (labels != ignore_index)
    return labels.masked_fill(~mask, 0), mask.float()


def masked_sum_loss(losses: torch.Tensor, loss_mask: torch.Tensor, *, loss_weight: Optional[torch.Tensor] = None,
                    per_token: bool = False, num_microbatches: int = 1, cp_size: int = 1, dp_cp_group=None):
    """Returns (loss for backward, report dict)."""
    m = loss_mask.float().reshape(-1)
    l = losses.float().reshape(-1)
    if loss_weight is not None:
        m = m * loss_weight.float().reshape(-1)
    total = (l * m).sum()
    count = m.sum()
    if per_token:
        # caller divides by the global token count after the all-reduce
        return total * cp_size, {"lm loss sum": total.detach(), "num_tokens": count.detach()}
    loss = total / count.clamp_min(1) * cp_size / num_microbatches
    return loss, {"lm loss": (total / count.clamp_min(1)).detach()}


def check_loss(loss_value: float, *, spiky_factor: float = 10.0, running_mean: Optional[float] = None) -> Optional[str]:
    """Loss validation used by the rerun machinery: returns 'nan', 'inf', 'spiky' or None."""
    if math.isnan(loss_value):
        return "nan"
    if math.isinf(loss_value):
        return "inf"
    if running_mean is not None and running_mean > 0 and loss_value > spiky_factor * running_mean:
        return "spiky"
    return None


def average_losses_across_data_parallel_group(values: Dict[str, torch.Tensor], group) -> Dict[str, float]:
    keys = sorted(values)
    t = torch.stack([values[k].float() for k in keys])
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, group=group)
        t /= dist.get_world_size(group)
    return dict(zip(keys, t.tolist()))
