"""Layer micro-benchmark that feeds the adaptive-FP8 policy: times forward + backward of the parallel linear layers of
a model (QKV, proj, FC1, FC2, expert FC1 / FC2) at a range of token counts in bf16 and in blockwise FP8, and exports
the policy JSON that ``runtime/fp8_policy.py`` reads (reference: tools/benchmark_te_parallel_layers.py:1-1610).

    python -m tools.benchmark_parallel_layers --model-name llama3-8b --tp 1 2 --tokens 1024 4096 16384 \
        --out policy.json [--csv rows.csv] [--markdown report.md] [--native-fp8]

Every linear kind the policy knows is covered: dense attention / MLP projections, the multi-latent-attention down / up
projections, the MTP projection, the output layer, routed experts (one grouped launch over the experts a rank holds,
tokens spread evenly over them) and shared experts. Each row has the forward and the forward + backward time of the
bf16 layer and of the FP8 layer as the trainer would run it (``ops/quant.py::fp8_linear``: block quantisation of
activations and weights included; ``--native-fp8`` turns the tcgen05 FP8 kernels on, otherwise the PyTorch formulation
runs), and the speed-up. Several ``--tp`` values are swept in one run; the exported policy has one rule per
(kind, tp) with the smallest token count from which FP8 wins by ``--min-speedup`` at every larger measured size.
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


def layer_shapes(cfg, tp: int, ep: int = 1) -> Dict[str, tuple]:
    """kind -> (in_features, out_features[, experts on this rank]) of the LOCAL shard."""
    h = cfg.hidden_size
    glu = 2 if cfg.gated_linear_unit else 1
    shapes: Dict[str, tuple] = {}
    if getattr(cfg, "multi_latent_attention", False):
        H = cfg.num_attention_heads
        qk = cfg.qk_head_dim + cfg.qk_pos_emb_head_dim
        if cfg.q_lora_rank:
            shapes["linear_q_down_proj"] = (h, cfg.q_lora_rank)
            shapes["linear_q_up_proj"] = (cfg.q_lora_rank, H * qk // tp)
        shapes["linear_kv_down_proj"] = (h, cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim)
        shapes["linear_kv_up_proj"] = (cfg.kv_lora_rank, H * (cfg.qk_head_dim + cfg.v_head_dim) // tp)
        shapes["linear_proj"] = (H * cfg.v_head_dim // tp, h)
    else:
        qkv = (cfg.num_attention_heads + 2 * cfg.num_query_groups) * cfg.kv_channels
        shapes["linear_qkv"] = (h, qkv // tp)
        shapes["linear_proj"] = (cfg.num_attention_heads * cfg.kv_channels // tp, h)
    shapes["linear_fc1"] = (h, glu * cfg.ffn_hidden_size // tp)
    shapes["linear_fc2"] = (cfg.ffn_hidden_size // tp, h)
    if cfg.num_moe_experts:
        local = max(1, cfg.num_moe_experts // max(ep, 1))
        shapes["experts.linear_fc1"] = (h, glu * cfg.moe_ffn_hidden_size, local)
        shapes["experts.linear_fc2"] = (cfg.moe_ffn_hidden_size, h, local)
        if cfg.moe_shared_expert_intermediate_size:
            shapes["shared_experts.linear_fc1"] = (h, glu * cfg.moe_shared_expert_intermediate_size // tp)
            shapes["shared_experts.linear_fc2"] = (cfg.moe_shared_expert_intermediate_size // tp, h)
    if getattr(cfg, "mtp_num_layers", 0):
        shapes["eh_proj"] = (2 * h, h)
    shapes["output_layer"] = (h, cfg.padded_vocab_size // tp if cfg.padded_vocab_size else cfg.vocab_size // tp)
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


def bench_layer(in_f: int, out_f: int, tokens: int, device, dtype, warmup: int = 3, iters: int = 10,
                experts: int = 0, topk: int = 1) -> Dict[str, float]:
    """One row: forward and forward + backward times of the bf16 and the FP8 layer. `experts` > 0: a grouped launch
    over that many experts with ``tokens * topk`` routed rows spread evenly."""
    from loongforge_b200.ops import functional as OF
    from loongforge_b200.ops import quant as Q

    cuda = torch.device(device).type == "cuda"
    rows = tokens * max(topk, 1) if experts else tokens
    x = torch.randn(rows, in_f, device=device, dtype=dtype, requires_grad=True)
    gy = torch.randn(rows, out_f, device=device, dtype=dtype)
    if experts:
        ws = [(torch.randn(out_f, in_f, device=device, dtype=dtype) * 0.02).requires_grad_() for _ in range(experts)]
        tpe = [rows // experts + (1 if i < rows % experts else 0) for i in range(experts)]

        def fwd(lin):
            return torch.cat([lin(xs, w) for xs, w in zip(x.split(tpe), ws)]) if not (cuda and lin is OF.linear) \
                else _grouped(x, ws, tpe)
        params = ws
    else:
        w = (torch.randn(out_f, in_f, device=device, dtype=dtype) * 0.02).requires_grad_()
        fwd = lambda lin: lin(x, w)  # noqa: E731
        params = [w]

    def _grouped(xx, weights, counts):
        from loongforge_b200.models.moe import GroupedLinear  # noqa: F401  (same kernel the expert layer launches)
        out = torch.empty(xx.shape[0], out_f, device=xx.device, dtype=xx.dtype)
        OF.grouped_gemm(xx.detach(), None, [p.detach() for p in weights], [out], counts, mode=0)
        return out.requires_grad_()

    def step(lin, backward):
        def run():
            x.grad = None
            for p in params:
                p.grad = None
            y = fwd(lin)
            if backward and y.grad_fn is not None:
                y.backward(gy)
        return run

    ok8 = Q.fp8_linear_supported(in_f, out_f)
    out = {"bf16_fwd_ms": _time(step(OF.linear, False), warmup, iters, cuda),
           "bf16_ms": _time(step(OF.linear, True), warmup, iters, cuda)}
    if ok8:
        out["fp8_fwd_ms"] = _time(step(Q.fp8_linear, False), warmup, iters, cuda)
        out["fp8_ms"] = _time(step(Q.fp8_linear, True), warmup, iters, cuda)
        out["speedup"] = out["bf16_ms"] / out["fp8_ms"]
    else:
        out.update(fp8_fwd_ms=float("inf"), fp8_ms=float("inf"), speedup=0.0)
    return out


def run(model_name: str, tp, token_counts: List[int], device=None, dtype=None, ep: int = 1, kinds=None, **kw) -> List[dict]:
    from loongforge_b200.models.registry import get_model_config

    cfg = get_model_config(model_name)
    cfg.pad_vocab(max(tp) if isinstance(tp, (list, tuple)) else tp)
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32)
    rows = []
    for t_p in (tp if isinstance(tp, (list, tuple)) else [tp]):
        for kind, shape in layer_shapes(cfg, t_p, ep).items():
            if kinds and kind not in kinds:
                continue
            in_f, out_f = shape[0], shape[1]
            experts = shape[2] if len(shape) > 2 else 0
            for t in token_counts:
                rows.append({"kind": kind, "tp": t_p, "tokens": t, "in_features": in_f, "out_features": out_f,
                             "experts": experts,
                             **bench_layer(in_f, out_f, t, device, dtype, experts=experts,
                                           topk=(cfg.moe_router_topk or 1) if experts else 1, **kw)})
    return rows


def to_markdown(rows: List[dict]) -> str:
    head = "| kind | tp | tokens | in x out | bf16 fwd / fwd+bwd ms | fp8 fwd / fwd+bwd ms | speed-up |\n|---|---|---|---|---|---|---|\n"
    fmt = lambda v: "-" if v == float("inf") else f"{v:.3f}"  # noqa: E731
    return head + "\n".join(
        f"| {r['kind']} | {r['tp']} | {r['tokens']} | {r['in_features']} x {r['out_features']}"
        f"{' x ' + str(r['experts']) + ' experts' if r['experts'] else ''} | {fmt(r['bf16_fwd_ms'])} / {fmt(r['bf16_ms'])} | "
        f"{fmt(r['fp8_fwd_ms'])} / {fmt(r['fp8_ms'])} | {r['speedup']:.2f} |" for r in rows) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", default="llama3-8b")
    ap.add_argument("--tp", type=int, nargs="+", default=[1])
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--tokens", type=int, nargs="+", default=[1024, 4096, 8192, 16384])
    ap.add_argument("--kinds", nargs="*", default=None, help="only these layer kinds")
    ap.add_argument("--min-speedup", type=float, default=1.05)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--native-fp8", action="store_true", help="FP8 quantisers and GEMM on the tcgen05 kernels")
    ap.add_argument("--out", default=None, help="policy JSON for --fp8-dynamic-policy-path")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--markdown", default=None)
    a = ap.parse_args(argv)
    from loongforge_b200.runtime.fp8_policy import export_policy_from_benchmark

    if a.native_fp8:
        from loongforge_b200.ops import quant as Q
        Q.enable_native(True)
    rows = run(a.model_name, a.tp, a.tokens, ep=a.ep, kinds=a.kinds, warmup=a.warmup, iters=a.iters)
    policy = export_policy_from_benchmark([r for r in rows if r["fp8_ms"] != float("inf")], a.min_speedup)
    out = {"rows": rows, "policy": policy}
    if a.csv:
        import csv
        with open(a.csv, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0]))
            wr.writeheader()
            wr.writerows(rows)
    if a.markdown:
        with open(a.markdown, "w") as f:
            f.write(to_markdown(rows))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(policy, f, indent=1)
    else:
        print(json.dumps(out, indent=1))
    return out


if __name__ == "__main__":
    main()
