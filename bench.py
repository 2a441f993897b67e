#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B-architecture dense pre-training, bf16, seq 8192.

    python bench.py --gpus N --steps K --warmup W            (N == 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W   (N > 1)

Parallel layout per N (weak scaling: 16 sequences of 8192 tokens per GPU and step, i.e. the
named global batch 128 at N = 8): N=1 -> TP1; N=2 -> TP2+SP; N=4 -> TP2+SP x DP2; N=8 -> TP2+SP x
DP4 with the distributed optimizer. Rank 0 prints ONE JSON line.

Two timed regions of K steps each, after W warm-up steps:
  * device-timed: CUDA events on the launching stream, barrier + synchronize on both sides, max
    over ranks; inputs already on the device -> ``value`` (whole-job tokens/s).
  * end-to-end: the same public call (``Trainer.train_step``) fed from pinned HOST memory
    (host->device copy of every micro-batch inside the step) and reading the loss back
    (device->host) every step -> ``e2e``.
No work is skipped: every step runs forward, backward, gradient reduction, clipping, AdamW and
the parameter refresh of the full 32-layer model.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Published per-GPU throughput of the reference for Llama3-8B pre-training (its CI baseline on
# the fastest chip it lists, 8 GPUs, seq 4096): tests/llm_vlm/baseline/default/BZZ/llama3_8b.json.
REF_PUBLISHED_TOK_S_GPU = 3550.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--seqs-per-gpu", type=int, default=16)
    ap.add_argument("--layers", type=int, default=32, help="debug only; anything but 32 is not the named config")
    ap.add_argument("--model", default="llama3-8b", help="registry preset; anything but llama3-8b is a side benchmark")
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--moe-dispatcher", default="alltoall", choices=["peer", "alltoall"])
    ap.add_argument("--pp", type=int, default=1, help="side benchmark: pipeline-parallel size")
    ap.add_argument("--images-per-sample", type=int, default=4, help="vision-language side benchmark")
    ap.add_argument("--encoder-hetero-dp", action="store_true",
                    help="vision-language side benchmark: images of a micro-batch split over the decoder's TP ranks")
    ap.add_argument("--full-hetero-dp", action="store_true",
                    help="vision-language side benchmark: all encoder rounds before the pipeline, one owner rank per micro-batch")
    ap.add_argument("--experts", type=int, default=None,
                    help="side benchmark: number of routed experts (e.g. the 32 a rank holds of DeepSeek's 256 at EP8)")
    ap.add_argument("--cp", type=int, default=1, help="side benchmark: context-parallel size")
    ap.add_argument("--no-fp8", action="store_true", help="side benchmark: run a preset that names fp8 in bf16")
    ap.add_argument("--overlap-moe-a2a", action="store_true",
                    help="MoE side benchmark: 1F1B interleave of expert-parallel exchanges with compute")
    ap.add_argument("--peer-optimizer", action="store_true",
                    help="gradient reduce-scatter / parameter all-gather inside the optimizer kernels over peer memory")
    ap.add_argument("--attention", default="auto", choices=["auto", "native", "sdpa"])
    ap.add_argument("--recompute", default="auto", choices=["auto", "none", "full"])
    ap.add_argument("--no-tp-overlap", action="store_true")
    ap.add_argument("--recompute-layers", type=int, default=None, help="with --recompute full: first K layers only")
    ap.add_argument("--fp32-master-copy", action="store_true",
                    help="keep a separate fp32 master tensor instead of the exact (bf16, int16 remainder) pair")
    return ap.parse_args()


def reference_arm(args):
    """The reference needs Loong-Megatron (an empty git submodule in its tree), TransformerEngine
    built from source and hydra/omegaconf; none exist offline, so its trainer cannot start."""
    why = ("reference not runnable offline: third_party/Loong-Megatron is an empty submodule "
           "(all megatron.* imports fail), TransformerEngine/hydra/omegaconf absent from the image")
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import importlib
        importlib.import_module("loongforge.train")
        why = "reference imported but cannot train: megatron runtime missing"
    except Exception as e:  # noqa: BLE001
        why += f" ({type(e).__name__}: {str(e)[:80]})"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.ops import _ext
    from loongforge_b200.ops import functional as OF
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer, init_distributed

    dev = init_distributed()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert dev.type == "cuda", "bench.py needs a GPU"
    _ext.require()
    OF.set_attention_impl(args.attention)

    flagship = args.model == "llama3-8b"
    tp = args.tp if args.tp is not None else (2 if world >= 2 and flagship else 1)
    dp = world // (tp * args.cp * args.pp)
    vlm = args.model in ("qwen2.5-vl-7b", "qwen2_5_vl_7b")
    if vlm:
        # Qwen2.5-VL-7B: Qwen2.5-7B language model with multimodal rotary positions + the 32-layer window-attention ViT
        cfg = get_model_config("qwen2.5-7b", position_embedding_type="mrope", mrope_section=[16, 24, 24])
    else:
        cfg = get_model_config(args.model)
    if vlm:
        pass
    elif flagship or args.layers != 32:
        cfg.num_layers = args.layers
    if cfg.num_moe_experts:
        cfg.moe_token_dispatcher_type = args.moe_dispatcher
        if args.experts:
            cfg.num_moe_experts = args.experts
            if cfg.moe_router_num_groups and args.experts % cfg.moe_router_num_groups:
                cfg.moe_router_num_groups = cfg.moe_router_group_topk = None
    if args.no_fp8:
        cfg.fp8 = None
    cfg.sequence_parallel = tp > 1
    cfg.tp_comm_overlap = tp > 1 and not args.no_tp_overlap
    # One GPU holds all 8 B parameters with exact fp32 master weights (bf16 + int16 remainder), fp32
    # Adam moments and fp32 gradient accumulation (~112 GB) plus ~30 GB of activations (the fused
    # norm+linear / swiglu+linear blocks recompute their cheap elementwise parts): 144 GB of 180 GB, so
    # no layer is recomputed at any N.
    recompute = args.recompute
    if recompute == "auto":
        recompute = "none"
    if recompute == "full":
        cfg.recompute_granularity, cfg.recompute_method = "full", "uniform"
        if args.recompute_layers is not None:
            cfg.recompute_method, cfg.recompute_num_layers = "block", args.recompute_layers
    gbs = args.seqs_per_gpu * world
    tc = TrainConfig(micro_batch_size=1, global_batch_size=gbs, seq_length=args.seq_len,
                     train_iters=10 ** 9, lr=3e-4, weight_decay=0.1, adam_beta2=0.95, clip_grad=1.0, bf16=True,
                     use_distributed_optimizer=True, overlap_grad_reduce=True,
                     master_as_remainder=not args.fp32_master_copy, peer_optimizer=args.peer_optimizer,
                     overlap_moe_expert_parallel_comm=args.overlap_moe_a2a)
    dims = ParallelDims(tp=tp, ep=args.ep, cp=args.cp, pp=args.pp)
    if vlm:
        from loongforge_b200.runtime.vlm import VLMTrainer, synthetic_vlm_iterator
        trainer = VLMTrainer(cfg, tc, dims, vit_cfg=get_model_config("qwen2.5-vit"), encoder_tp=1, encoder_recompute=True,
                             encoder_hetero_dp=args.encoder_hetero_dp, full_hetero_dp=args.full_hetero_dp,
                             images_per_sample=args.images_per_sample, image_size=448, device=dev)
        st = trainer.st
        host_iter = synthetic_vlm_iterator(cfg.vocab_size, tc.seq_length, images_per_sample=args.images_per_sample,
                                           image_size=448, dp_rank=st.dp_rank, dp_size=st.dp_size, pin_memory=True)
    else:
        trainer = Trainer(cfg, tc, dims, device=dev)
        st = trainer.st
        host_iter = synthetic_batch_iterator(cfg.vocab_size, tc.seq_length, 1, dp_rank=st.dp_rank, dp_size=st.dp_size,
                                             pin_memory=True)

    def device_iter():
        # the same synthetic stream, staged on the device ahead of time (device-timed region)
        cache = []
        for _ in range(trainer.mb_calc.num_microbatches):
            b = next(host_iter)
            cache.append({k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in b.items()})
        while True:
            for b in cache:
                yield b

    dit = device_iter()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.train_step(dit)
    _ext.check_status()

    # ---------------------------------------------------------------- device-timed region
    sampler = ClockSampler(dev.index or 0)
    barrier()
    sampler.start()
    _ext.reset_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        m = trainer.train_step(dit)
    ev1.record()
    barrier()
    launches = _ext.launch_count()
    dev_ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop()

    # ---------------------------------------------------------------- end-to-end region
    h2d = 0
    barrier()
    t0 = time.perf_counter()
    last_loss = None
    for _ in range(args.steps):
        m = trainer.train_step(host_iter)  # H2D of every micro-batch inside; loss read back (D2H)
        last_loss = m.get("lm loss")
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    _ext.check_status()
    per_mb = tc.seq_length * (8 + 8 + 4 + 8)  # tokens, labels (int64), loss_mask (fp32), position ids (int64)
    h2d = per_mb * trainer.mb_calc.num_microbatches
    d2h = 8 + 4  # loss scalar (fp32 metrics vector) + grad-norm scalar

    t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    tokens_per_step = gbs * tc.seq_length
    ms_per_step = dev_ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    e2e_value = tokens_per_step / (e2e_ms / args.steps / 1e3)
    flops = cfg.flops_per_token(tc.seq_length) * tokens_per_step
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:  # noqa: BLE001
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    tflops_gpu = flops / (ms_per_step / 1e3) / 1e12 / world
    if rank == 0:
        out = {
            "metric": ("tokens/sec (whole job) on Llama-3-8B pretrain; per-GPU and MFU in config" if flagship else
                       f"tokens/sec (whole job) on {args.model} pretrain (side benchmark)"),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / world) / REF_PUBLISHED_TOK_S_GPU if flagship else None,
            "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights", "impl": "ours",
            "config": {
                "model": (f"llama3-8b ({cfg.num_layers} layers, h4096, 32q/8kv, ffn14336, vocab128256)" if flagship else
                          f"{args.model} ({cfg.num_layers} layers, ep{args.ep}, dispatcher {args.moe_dispatcher})"),
                "global_batch": gbs, "seq_len": tc.seq_length, "micro_batch": 1,
                "parallelism": (f"tp{tp}+sp" if tp > 1 else "tp1") + (f" pp{args.pp}" if args.pp > 1 else "")
                + (f" cp{args.cp}" if args.cp > 1 else "") + f" dp{dp} distributed-optimizer",
                "recompute": recompute, "attention_impl": args.attention,
                "tp_comm_overlap": bool(cfg.tp_comm_overlap),
                "tokens_per_sec_per_gpu": value / world, "model_tflops_per_gpu": tflops_gpu,
                "mfu_of_measured_sustained_bf16": tflops_gpu / peak,
                "l2_policy": "inputs larger than L2: 16 GB of weights + activations stream every step",
                "baseline_number": "3550 tok/s/GPU (reference CI, 8 x BZZ chip, seq 4096, TP2 PP2 CP2)",
                "last_loss": last_loss,
                "fp32_master": "separate fp32 tensor" if args.fp32_master_copy else "exact (bf16, int16 remainder) pair",
                "max_memory_allocated_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
            },
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
