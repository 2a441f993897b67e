"""Layer micro-benchmark that feeds the adaptive-FP8 policy: times forward + backward of the parallel linear layers of
a model (QKV, proj, FC1, FC2, expert FC1 / FC2) at a range of token counts in bf16 and in blockwise FP8, and exports
the policy JSON that ``runtime/fp8_policy.py`` reads (reference: tools/benchmark_te_parallel_layers.py:1-1610).

    python -m tools.benchmark_parallel_layers --model-name llama3-8b --tp 2 --tokens 1024 4096 16384 --out policy.json

Timing uses CUDA events after warm-up on a GPU (perf_counter on CPU, for the tool's own tests)."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, List

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402


def layer_shapes(cfg, tp: int) -> Dict[str, tuple]:
    """kind -> (in_features, out_features) of the LOCAL shard."""
    h = cfg.hidden_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_query_groups) * cfg.kv_channels
    glu = 2 if cfg.gated_linear_unit else 1
    shapes = {"linear_qkv": (h, qkv // tp), "linear_proj": (cfg.num_attention_heads * cfg.kv_channels // tp, h),
              "linear_fc1": (h, glu * cfg.ffn_hidden_size // tp), "linear_fc2": (cfg.ffn_hidden_size // tp, h)}
    if cfg.num_moe_experts:
        shapes["experts.linear_fc1"] = (h, glu * cfg.moe_ffn_hidden_size)
        shapes["experts.linear_fc2"] = (cfg.moe_ffn_hidden_size, h)
    return shapes


def _time(fn, warmup: int, iters: int, cuda: bool) -> float:
    for _ in range(warmup):
        fn()
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) * 1e3 / iters


def bench_layer(in_f: int, out_f: int, tokens: int, device, dtype, warmup: int = 3, iters: int = 10) -> Dict[str, float]:
    from loongforge_b200.ops import functional as OF
    from loongforge_b200.ops import quant as Q

    cuda = torch.device(device).type == "cuda"
    x = torch.randn(tokens, in_f, device=device, dtype=dtype, requires_grad=True)
    w = (torch.randn(out_f, in_f, device=device, dtype=dtype) * 0.02).requires_grad_()
    gy = torch.randn(tokens, out_f, device=device, dtype=dtype)

    def bf16_step():
        x.grad = w.grad = None
        OF.linear(x, w).backward(gy)

    def fp8_step():
        # forward in FP8 (both operands block-quantised); backward GEMMs on the de-quantised operands
        with torch.no_grad():
            Q.fp8_blockwise_linear(x, w)
        x.grad = w.grad = None
        OF.linear(x, w).backward(gy)

    ok8 = in_f % 128 == 0 and out_f % 128 == 0
    return {"bf16_ms": _time(bf16_step, warmup, iters, cuda),
            "fp8_ms": _time(fp8_step, warmup, iters, cuda) if ok8 else float("inf")}


def run(model_name: str, tp: int, token_counts: List[int], device=None, dtype=None, **kw) -> List[dict]:
    from loongforge_b200.models.registry import get_model_config

    cfg = get_model_config(model_name)
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32)
    rows = []
    for kind, (in_f, out_f) in layer_shapes(cfg, tp).items():
        for t in token_counts:
            rows.append({"kind": kind, "tp": tp, "tokens": t, "in_features": in_f, "out_features": out_f,
                         **bench_layer(in_f, out_f, t, device, dtype, **kw)})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-name", default="llama3-8b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--tokens", type=int, nargs="+", default=[1024, 4096, 8192, 16384])
    ap.add_argument("--min-speedup", type=float, default=1.05)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    from loongforge_b200.runtime.fp8_policy import export_policy_from_benchmark

    rows = run(a.model_name, a.tp, a.tokens)
    policy = export_policy_from_benchmark([r for r in rows if r["fp8_ms"] != float("inf")], a.min_speedup)
    out = {"rows": rows, "policy": policy}
    if a.out:
        with open(a.out, "w") as f:
            json.dump(policy, f, indent=1)
    else:
        print(json.dumps(out, indent=1))
    return out


if __name__ == "__main__":
    main()
