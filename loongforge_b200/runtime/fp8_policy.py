"""Adaptive (selective) FP8: a JSON policy decides per linear-layer KIND, token count and tensor-parallel size whether
that module runs its GEMMs in FP8 or stays in BF16, because small or skinny GEMMs lose more in quantisation overhead
than they gain (reference: loongforge/train/fp8_dynamic_policy.py:63-281; the policy file is produced by a layer
benchmark, reference tools/benchmark_te_parallel_layers.py).

Policy file::

    {"default": "bf16",
     "rules": [{"kind": "linear_fc1", "min_tokens": 4096, "tp": [1, 2], "precision": "fp8"},
               {"kind": "linear_qkv", "min_tokens": 8192, "precision": "fp8"}]}

Rules are tried in order; the first whose kind matches (glob) and whose token / tp / shape bounds hold wins.
"""
from __future__ import annotations

import dataclasses
import fnmatch
import json
from typing import Dict, List, Optional

import torch.nn as nn

LINEAR_KINDS = ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2", "linear_q_down_proj", "linear_q_up_proj",
                "linear_kv_down_proj", "linear_kv_up_proj", "eh_proj", "output_layer", "experts.linear_fc1",
                "experts.linear_fc2", "shared_experts.linear_fc1", "shared_experts.linear_fc2")


@dataclasses.dataclass
class Rule:
    kind: str
    precision: str
    min_tokens: int = 0
    max_tokens: Optional[int] = None
    tp: Optional[List[int]] = None
    min_in_features: int = 0
    min_out_features: int = 0

    def matches(self, kind: str, tokens: int, tp: int, in_f: int, out_f: int) -> bool:
        return (fnmatch.fnmatch(kind, self.kind) and tokens >= self.min_tokens
                and (self.max_tokens is None or tokens <= self.max_tokens) and (self.tp is None or tp in self.tp)
                and in_f >= self.min_in_features and out_f >= self.min_out_features)


class FP8Policy:
    def __init__(self, rules: List[Rule], default: str = "bf16"):
        self.rules, self.default = rules, default

    @staticmethod
    def from_json(path_or_dict) -> "FP8Policy":
        d = path_or_dict
        if not isinstance(d, dict):
            with open(path_or_dict) as f:
                d = json.load(f)
        for r in d.get("rules", []):
            if r["precision"] not in ("fp8", "bf16"):
                raise ValueError(f"unknown precision {r['precision']!r}")
        return FP8Policy([Rule(**r) for r in d.get("rules", [])], d.get("default", "bf16"))

    def decide(self, kind: str, tokens: int, tp: int, in_features: int, out_features: int) -> str:
        for r in self.rules:
            if r.matches(kind, tokens, tp, in_features, out_features):
                return r.precision
        return self.default


def module_kind(qualified_name: str) -> Optional[str]:
    """``decoder.layers.3.mlp.experts.linear_fc1`` -> ``experts.linear_fc1``; None for non-linear modules."""
    best = None
    for k in LINEAR_KINDS:
        if qualified_name == k or qualified_name.endswith("." + k):
            if best is None or len(k) > len(best):
                best = k
    return best


def apply_fp8_policy(model: nn.Module, policy: FP8Policy, tokens_per_microbatch: int, tp: int) -> Dict[str, str]:
    """Sets ``module.gemm_precision`` ('fp8' | 'bf16') on every linear-like module at init time and returns the
    decisions. Linear layers consult the attribute when they pick their GEMM."""
    out = {}
    for name, mod in model.named_modules():
        kind = module_kind(name)
        if kind is None:
            continue
        w = getattr(mod, "weight", None)
        if w is None and hasattr(mod, "weights"):
            ws = mod.weights()
            w = ws[0] if ws else None
        if w is None or w.dim() != 2:
            continue
        prec = policy.decide(kind, tokens_per_microbatch, tp, w.shape[1], w.shape[0])
        if prec == "fp8" and not _can_run_fp8(mod, w):
            prec = "bf16"
        mod.gemm_precision = prec
        out[name] = prec
    return out


def _can_run_fp8(mod: nn.Module, w) -> bool:
    """FP8 GEMMs exist for the dense tensor-parallel linears on feature sizes that are multiples of the 128-wide
    quantisation block; grouped expert GEMMs and the kernels fused with tensor-parallel collectives run in bf16."""
    from ..ops.quant import fp8_linear_supported
    from ..parallel.layers import ColumnParallelLinear, RowParallelLinear

    if not isinstance(mod, (ColumnParallelLinear, RowParallelLinear)):
        return False
    if getattr(mod, "tp_comm_overlap", False) and getattr(mod, "tp", 1) > 1:
        return False
    return fp8_linear_supported(w.shape[1], w.shape[0])


def default_policy() -> FP8Policy:
    """Every transformer-layer linear in FP8; the output layer (logits) stays in bf16."""
    return FP8Policy([Rule(kind="output_layer", precision="bf16")], default="fp8")


def export_policy_from_benchmark(rows: List[dict], min_speedup: float = 1.05) -> dict:
    """Benchmark rows ``{kind, tokens, tp, bf16_ms, fp8_ms}`` -> policy: per (kind, tp) the smallest token count from
    which FP8 is at least `min_speedup` faster for every larger measured size."""
    by = {}
    for r in rows:
        by.setdefault((r["kind"], r["tp"]), []).append(r)
    rules = []
    for (kind, tp), rs in sorted(by.items()):
        rs.sort(key=lambda r: r["tokens"])
        thr = None
        for i, r in enumerate(rs):
            if all(x["bf16_ms"] / x["fp8_ms"] >= min_speedup for x in rs[i:]):
                thr = r["tokens"]
                break
        if thr is not None:
            rules.append({"kind": kind, "tp": [tp], "min_tokens": thr, "precision": "fp8"})
    return {"default": "bf16", "rules": rules}
