"""Micro-benchmarks of the native kernels (CUDA-event timing, warm-up, L2-exceeding inputs).

    python -m loongforge_b200.ops.bench_kernels gemm [--m 8192 --n 4096 --k 4096] [--iters 20]
    python -m loongforge_b200.ops.bench_kernels attention [--t 8192 --groups 8 --rep 4]
    python -m loongforge_b200.ops.bench_kernels norm [--t 8192 --h 4096]
    python -m loongforge_b200.ops.bench_kernels elementwise [--t 8192 --h 4096]   (RoPE, SwiGLU, linear + CE, AdamW)
    python -m loongforge_b200.ops.bench_kernels dsa [--t 4096 --skv 8192 --topk 2048 --impl ours|torch|reference]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        -m loongforge_b200.ops.bench_kernels tp [--t 8192]     (fused TP GEMMs against NCCL + GEMM, Llama-3-8B shapes)

Each sub-command prints one JSON line; `--once` runs a single un-timed invocation (for profilers).
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from . import _ext
from . import functional as OF


def _time(fn, iters, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def dsa_bench(a):
    """DeepSeek sparse attention kernels on the reference's own test shape (ops/tilelang_ops/sparse_mla_fwd.py:
    S queries x 128 heads x 576 dims against SKV keys, top-k 2048; indexer 64 heads x 128 dims): `ours` = the tcgen05
    kernels of csrc/dsa_sm100.cu, `torch` = the blocked PyTorch formulation, `reference` = the reference's TileLang
    kernels imported unmodified from a copy of its ops/ directory under baseline/_ref."""
    import os
    import sys

    from . import dsa_ops

    S, SKV, K, H = a.t, a.skv, a.topk if a.topk > 8 else 2048, 128
    dev = "cuda"
    torch.manual_seed(0)
    q = (torch.randn(S, H, 576, device=dev) * 0.3).bfloat16()
    kv = (torch.randn(SKV, 576, device=dev) * 0.3).bfloat16()
    # causal selection: query i sits at key position i + SKV - S and picks K of the keys it may see
    lim = torch.arange(S, device=dev) + (SKV - S) + 1
    idx = (torch.rand(S, K, device=dev) * lim[:, None]).int().clamp_(max=SKV - 1)
    idx = torch.where(torch.arange(K, device=dev)[None, :] < lim[:, None], idx, torch.full_like(idx, -1))
    scale = 576 ** -0.5
    qi = torch.randn(S, 64, 128, device=dev).bfloat16()
    ki = torch.randn(SKV, 128, device=dev).bfloat16()
    wi = torch.randn(S, 64, device=dev) * 0.1
    pos_q, pos_k = torch.arange(S, device=dev) + (SKV - S), torch.arange(SKV, device=dev)
    out = {"what": "dsa", "impl": a.impl, "s": S, "skv": SKV, "topk": K, "heads": H}
    fl_attn = 2.0 * S * K * H * (576 + 512) / 1e9          # useful FLOPs (one score pass)
    fl_idx = 2.0 * 64 * 128 * float((lim.clamp(max=SKV)).sum()) / 1e9
    if a.impl == "ours":
        C, st = _ext.require(), _ext.status_tensor(q.device)
        f_attn = lambda: C.sparse_mla_fwd(q, kv, idx, scale, st)  # noqa: E731
        f_idx = lambda: dsa_ops.indexer_topk(qi, ki, wi, K, pos_q, pos_k, keys_in_order=True)  # noqa: E731
    elif a.impl == "torch":
        f_attn = lambda: dsa_ops._sparse_mla_block(q[:256], idx[:256].long(), kv, scale, 512, False)  # noqa: E731
        f_idx = lambda: dsa_ops.indexer_topk(qi, ki, wi, K, pos_q, pos_k, keys_in_order=False)  # noqa: E731
        fl_attn *= 256.0 / S  # one 256-query block (what fits without the blockwise wrapper)
    else:
        ref = os.path.join(os.path.dirname(__file__), "..", "..", "baseline", "_ref", "ops", "tilelang_ops")
        if not os.path.isdir(ref):
            print(json.dumps({"what": "dsa", "impl": "reference", "unavailable": "baseline/_ref/ops/tilelang_ops missing"}))
            return
        sys.path.insert(0, os.path.abspath(ref))
        try:
            import sparse_mla_fwd as R  # the reference's file, unmodified
            offsets = torch.tensor([0, S], dtype=torch.int32, device=dev)  # query-token boundaries, as in its own test
            idx_r = idx.clone()
            idx_r[idx_r < 0] = SKV  # the reference marks unused slots with an index past the keys
            kv3, idx3 = kv.view(SKV, 1, 576).contiguous(), idx_r.view(S, 1, K).contiguous()
            f_attn = lambda: R.sparse_mla_fwd_interface(q, kv3, idx3, offsets, chunk_offset=SKV - S, sm_scale=scale,  # noqa: E731
                                                        block_I=64, num_stages=2, threads=256)
            f_attn()
            torch.cuda.synchronize()
        except Exception as e:  # noqa: BLE001 - the TileLang kernels may not build for this architecture
            print(json.dumps({"what": "dsa", "impl": "reference",
                              "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}))
            return
        f_idx = None
    if a.once:
        f_attn()
        if f_idx:
            f_idx()
    else:
        ms = _time(f_attn, a.iters, warm=2)
        out.update(sparse_mla_fwd_ms=ms, sparse_mla_fwd_tflops=fl_attn / ms)
        if f_idx:
            ms = _time(f_idx, max(2, a.iters // 4), warm=1)
            out.update(indexer_topk_ms=ms, indexer_logits_tflops=fl_idx / ms)
    torch.cuda.synchronize()
    _ext.check_status()
    print(json.dumps(out))


def tp_bench(a):
    """All-gather->GEMM and GEMM->reduce-scatter of one tensor-parallel Llama-3-8B layer (hidden 4096, FFN 14336,
    32 q / 8 kv heads) on `world` GPUs: the fused peer-memory kernels against NCCL collective + plain GEMM, forward
    shapes. Times are CUDA-event times, max over ranks; the roofline is the slower of the FLOPs at the measured
    sustained bf16 peak and the bytes that must cross NVLink at the measured 770 GB/s per direction."""
    import os

    import torch.distributed as dist

    from ..parallel import fused_tp, state as ps

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    ps.initialize_model_parallel(ps.ParallelDims(tp=world))
    g = ps.get_state().group("tp")
    T, H, F = a.t, 4096, 14336
    rows = T // world
    peak = 1376.9e12
    try:
        peak = json.load(open(os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")))[
            "bf16_tflops_sustained"] * 1e12
    except Exception:  # noqa: BLE001
        pass
    torch.manual_seed(0)
    res = {"what": "tp", "world": world, "t": T, "rows": []}

    def timed(fn):
        ms = torch.tensor([_time(fn, a.iters)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    # (name, kind, K, N_local)
    shapes = [("qkv", "ag", H, (32 + 16) * 128 // world), ("fc1", "ag", H, 2 * F // world),
              ("proj", "rs", H // world, H), ("fc2", "rs", F // world, H)]
    for name, kind, K, N in shapes:
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        if kind == "ag":
            xs = torch.randn(rows, K, device=dev).bfloat16()
            xf = torch.empty(T, K, device=dev, dtype=torch.bfloat16)

            def nccl():
                dist.all_gather_into_tensor(xf, xs, group=g)
                return OF.gemm(xf, w)

            fused = lambda: fused_tp._ag_gemm(xs, w, False, None, None)[0]  # noqa: E731
            link_bytes = (world - 1) * rows * K * 2  # received per GPU
        else:
            x = torch.randn(T, K, device=dev).bfloat16()
            out = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)

            def nccl():
                y = OF.gemm(x, w)
                dist.reduce_scatter_tensor(out, y, group=g)
                return out

            fused = lambda: fused_tp._gemm_rs(x, w, False, None, None)  # noqa: E731
            link_bytes = (world - 1) * rows * N * 2  # partial sums sent per GPU
        flops = 2.0 * T * K * N
        t_n, t_f = timed(nccl), timed(fused)
        t_gemm = timed((lambda: OF.gemm(xf, w)) if kind == "ag" else (lambda: OF.gemm(x, w)))
        ideal = max(flops / peak, link_bytes / 770e9) * 1e3
        res["rows"].append({"layer": name, "kind": kind, "K": K, "N": N, "nccl_plus_gemm_ms": t_n, "fused_ms": t_f,
                            "gemm_only_ms": t_gemm, "roofline_ms": ideal, "fused_fraction_of_roofline": ideal / t_f})
    torch.cuda.synchronize()
    _ext.check_status()
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attention", "norm", "grouped", "router", "fp8", "tp", "dsa", "elementwise"])
    ap.add_argument("--skv", type=int, default=8192)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch", "reference"])
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--t", type=int, default=8192)
    ap.add_argument("--h", type=int, default=4096)
    ap.add_argument("--groups", type=int, default=8)
    ap.add_argument("--rep", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    _ext.require()
    if a.what == "tp":
        return tp_bench(a)
    if a.what == "dsa":
        return dsa_bench(a)
    dev = "cuda"
    torch.manual_seed(0)
    out = {"what": a.what}
    if a.what == "gemm":
        A = torch.randn(a.m, a.k, device=dev).bfloat16()
        B = torch.randn(a.n, a.k, device=dev).bfloat16()
        dY = torch.randn(a.m, a.n, device=dev).bfloat16()
        mg = torch.zeros(a.n, a.k, device=dev)
        fns = {"fwd_nt": lambda: OF.gemm(A, B), "dgrad_nn": lambda: OF.gemm(dY, B, b_mn_major=True),
               "wgrad_tn_acc": lambda: OF.gemm(dY, A, a_mn_major=True, b_mn_major=True, out=mg, out_mode=2)}
        if a.once:
            for f in fns.values():
                f()
        else:
            fl = 2.0 * a.m * a.n * a.k / 1e9
            for k_, f in fns.items():
                out[k_ + "_tflops"] = fl / _time(f, a.iters)
            out["cublas_fwd_tflops"] = fl / _time(lambda: A @ B.t(), a.iters)
        out.update(m=a.m, n=a.n, k=a.k)
    elif a.what == "attention":
        G, R, T = a.groups, a.rep, a.t
        qkv = torch.randn(T, G * (R + 2) * 128, device=dev).bfloat16().requires_grad_()
        o = OF.attention_packed(qkv, G, R)
        do = torch.randn_like(o)

        def fb():
            oo = OF.attention_packed(qkv, G, R)
            oo.backward(do)
            qkv.grad = None

        if a.once:
            fb()
        else:
            fl = 4.0 * T * T * 128 * G * R / 2 / 1e9
            tf = _time(lambda: OF.attention_packed(qkv.detach(), G, R), a.iters)
            tfb = _time(fb, a.iters)
            out.update(fwd_ms=tf, fwd_tflops=fl / tf, bwd_ms=tfb - tf, bwd_tflops=2.5 * fl / (tfb - tf))
        out.update(t=T, q_heads=G * R, kv_heads=G)
    elif a.what == "grouped":
        # E experts with m / E rows each (ragged by +-25 %), weights [n, k]: forward, dgrad, wgrad (fp32 accumulate)
        E = a.experts
        gen = torch.Generator().manual_seed(0)
        base = a.m // E
        tpe = [max(1, int(base * (0.75 + 0.5 * float(torch.rand(1, generator=gen))))) for _ in range(E)]
        T = sum(tpe)
        X = torch.randn(T, a.k, device=dev).bfloat16()
        dY = torch.randn(T, a.n, device=dev).bfloat16()
        Y, dX = torch.empty(T, a.n, device=dev).bfloat16(), torch.empty(T, a.k, device=dev).bfloat16()
        W = [(torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16() for _ in range(E)]
        MG = [torch.zeros(a.n, a.k, device=dev) for _ in range(E)]
        fns = {"fwd": lambda: OF.grouped_gemm(X, None, W, [Y], tpe, mode=0),
               "dgrad": lambda: OF.grouped_gemm(dY, None, W, [dX], tpe, mode=1),
               "wgrad_acc": lambda: OF.grouped_gemm(dY, X, [], MG, tpe, mode=2, out_mode=2)}
        if a.once:
            for f in fns.values():
                f()
        else:
            fl = 2.0 * T * a.n * a.k / 1e9
            for k_, f in fns.items():
                out[k_ + "_tflops"] = fl / _time(f, a.iters)
        out.update(experts=E, rows=T, n=a.n, k=a.k)
    elif a.what == "router":
        from . import moe_ops
        logits = torch.randn(a.t, a.experts, device=dev)
        f = lambda: moe_ops.topk_routing(logits, a.topk)  # noqa: E731
        if a.once:
            f()
        else:
            ms = _time(f, a.iters)
            out.update(ms=ms, gbytes_per_s=a.t * a.experts * (4 + 4 + 4 + 1) / ms / 1e6)
        out.update(t=a.t, experts=a.experts, topk=a.topk)
    elif a.what == "elementwise":
        # memory-bound ops of one Llama-3-8B layer / step at `t` tokens: achieved bytes per second against the copy peak
        T, H, F, V = a.t, a.h, 14336, 32064
        qkv = torch.randn(T, 48 * 128, device=dev).bfloat16()  # packed QKV: 8 groups of (4 q + k + v) heads
        freqs = OF.rope_freqs(torch.arange(T, device=dev), 128, 500000.0)
        hf = torch.randn(T, 2 * F, device=dev).bfloat16().requires_grad_()
        gf = torch.randn(T, F, device=dev).bfloat16()
        hid = torch.randn(T, H, device=dev).bfloat16().requires_grad_()
        wv = (torch.randn(V, H, device=dev) * 0.02).bfloat16().requires_grad_()
        labels = torch.randint(0, V, (T,), device=dev)
        mask = torch.ones(T, device=dev)
        n = 64 * 1024 * 1024  # one optimizer shard of 64 Mi parameters
        w16, lo = torch.randn(n, device=dev).bfloat16(), torch.zeros(n, dtype=torch.int16, device=dev)
        grad, m1, m2 = torch.randn(n, device=dev) * 1e-3, torch.zeros(n, device=dev), torch.zeros(n, device=dev)

        def f_rope():
            OF.rope(qkv, freqs, group=6, rope_in_group=5, inplace=True, head_dim=128)

        def f_swiglu():
            y = OF.swiglu(hf)
            y.backward(gf)
            hf.grad = None

        def f_ce():
            los = OF.linear_cross_entropy(hid, wv, labels, mask)
            ((los * mask).sum() / T).backward()
            hid.grad = None
            wv.grad = None

        def f_adam():
            OF.adam_step_remainder(w16, lo, grad, m1, m2, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                   step=3)

        fns = {"rope": (f_rope, T * 48 * 128 * 2 * 2 * 5 / 6), "swiglu_fwd_bwd": (f_swiglu, T * F * 2 * (3 + 5)),
               "adamw_remainder": (f_adam, n * (2 + 2 + 4 + 4 + 4) * 1.0 + n * (2 + 2 + 4 + 4))}
        if a.once:
            for f, _ in fns.values():
                f()
            f_ce()
        else:
            for k_, (f, nbytes) in fns.items():
                ms = _time(f, a.iters)
                out[k_ + "_ms"] = ms
                out[k_ + "_gbytes_per_s"] = nbytes / ms / 1e6
            ms = _time(f_ce, max(2, a.iters // 4), warm=2)
            out["linear_ce_fwd_bwd_ms"] = ms
            out["linear_ce_tflops"] = 3 * 2.0 * T * H * V / ms / 1e9  # logits, dgrad, wgrad
        out.update(t=T, h=H, ffn=F, vocab=V, adam_params=n)
    elif a.what == "fp8":
        from . import quant as Q
        Q.enable_native(True)
        x = torch.randn(a.m, a.k, device=dev).bfloat16()
        w = (torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16()
        qx, sx = Q.quantize_1x128(x)
        qw, sw = Q.quantize_128x128(w)
        C = _ext.require()
        st = _ext.status_tensor(x.device)
        fns = {"quant_1x128": lambda: Q.quantize_1x128(x), "quant_128x128": lambda: Q.quantize_128x128(w),
               "gemm": lambda: C.gemm_fp8_blockwise(qx, sx, qw, sw, st)}
        if a.once:
            for f in fns.values():
                f()
        else:
            out["quant_1x128_gbytes_per_s"] = a.m * a.k * 3 / _time(fns["quant_1x128"], a.iters) / 1e6
            out["quant_128x128_gbytes_per_s"] = a.n * a.k * 3 / _time(fns["quant_128x128"], a.iters) / 1e6
            out["gemm_tflops"] = 2.0 * a.m * a.n * a.k / 1e9 / _time(fns["gemm"], a.iters)
            out["bf16_gemm_tflops"] = 2.0 * a.m * a.n * a.k / 1e9 / _time(lambda: OF.gemm(x, w), a.iters)
        out.update(m=a.m, n=a.n, k=a.k)
    else:
        x = torch.randn(a.t, a.h, device=dev).bfloat16().requires_grad_()
        w = torch.ones(a.h, device=dev).bfloat16().requires_grad_()
        g = torch.randn(a.t, a.h, device=dev).bfloat16()

        def fb():
            y = OF.rmsnorm(x, w, 1e-5)
            y.backward(g)
            x.grad = None
            w.grad = None

        if a.once:
            fb()
        else:
            ms = _time(fb, a.iters)
            out.update(fwd_bwd_ms=ms, gbytes_per_s=a.t * a.h * 2 * 5 / ms / 1e6)
    torch.cuda.synchronize()
    _ext.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
