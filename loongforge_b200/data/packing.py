"""Sequence packing for SFT: greedy first-fit-decreasing bins (the reference's offline hash-bucket
packer and online packer, tools/data_preprocess/** and loongforge/train/sft/utils.py:330-972), and
the longest-processing-time partition used to balance packed groups across ranks."""
from __future__ import annotations

import heapq
from typing import Dict, List, Sequence, Tuple

import torch


def pack_first_fit_decreasing(lengths: Sequence[int], capacity: int) -> List[List[int]]:
    """Bins of sample indices with total length <= capacity (samples longer than capacity get their own bin)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[List[int]] = []
    free: List[int] = []
    for i in order:
        n = min(lengths[i], capacity)
        for b, f in enumerate(free):
            if n <= f:
                bins[b].append(i)
                free[b] -= n
                break
        else:
            bins.append([i])
            free.append(capacity - n)
    return bins


def lpt_partition(costs: Sequence[float], parts: int) -> List[List[int]]:
    """Longest-processing-time-first assignment of items to `parts` groups with balanced total cost."""
    heap = [(0.0, p) for p in range(parts)]
    heapq.heapify(heap)
    groups: List[List[int]] = [[] for _ in range(parts)]
    for i in sorted(range(len(costs)), key=lambda j: -costs[j]):
        load, p = heapq.heappop(heap)
        groups[p].append(i)
        heapq.heappush(heap, (load + costs[i], p))
    return groups


def collate_packed(samples: List[Tuple[List[int], List[int]]], capacity: int, pad_id: int = 0,
                   pad_to_multiple: int = 1) -> Dict[str, torch.Tensor]:
    """Concatenate (input_ids, labels) pairs into ONE packed row: tokens, shifted labels, loss mask,
    per-sequence position ids and ``cu_seqlens`` (padding forms a final dummy sequence)."""
    toks, labs, pos, cu = [], [], [], [0]
    for ids, lab in samples:
        ids, lab = ids[:capacity - len(toks)], lab[:capacity - len(toks)]
        if len(ids) < 2:
            continue
        toks.extend(ids)
        labs.extend(lab[1:] + [-100])  # next-token targets; the last token of a sample predicts nothing
        pos.extend(range(len(ids)))
        cu.append(len(toks))
    total = len(toks)
    target = capacity if pad_to_multiple <= 1 else min(capacity, -(-total // pad_to_multiple) * pad_to_multiple)
    target = max(target, total)
    if target > total:
        pad = target - total
        toks.extend([pad_id] * pad)
        labs.extend([-100] * pad)
        pos.extend(range(pad))
        cu.append(target)
    labels = torch.tensor(labs, dtype=torch.long)
    mask = (labels != -100).float()
    return {"tokens": torch.tensor(toks, dtype=torch.long).unsqueeze(0),
            "labels": labels.clamp_min(0).unsqueeze(0), "loss_mask": mask.unsqueeze(0),
            "position_ids": torch.tensor(pos, dtype=torch.long).unsqueeze(0),
            "cu_seqlens": torch.tensor(cu, dtype=torch.int32), "num_valid_tokens": int(mask.sum().item())}
