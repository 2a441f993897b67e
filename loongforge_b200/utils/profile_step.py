"""Kernel-time shares of one training step via torch.profiler: ``python -m loongforge_b200.utils.profile_step
--model NAME --layers L --seq-len S --seqs B``. Times taken under the profiler are for comparing SHARES between
kernels, never a benchmark value."""
import argparse, os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
from torch.profiler import profile, ProfilerActivity


def main():

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--seqs", type=int, default=2)
    ap.add_argument("--dispatcher", default="peer")
    ap.add_argument("--rows", type=int, default=45)
    args = ap.parse_args()
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer, init_distributed
    dev = init_distributed()
    cfg = get_model_config(args.model)
    cfg.num_layers = args.layers
    if cfg.num_moe_experts:
        cfg.moe_token_dispatcher_type = args.dispatcher
    tc = TrainConfig(micro_batch_size=1, global_batch_size=args.seqs, seq_length=args.seq_len, train_iters=10**9, lr=3e-4,
                     weight_decay=0.1, clip_grad=1.0, bf16=True, use_distributed_optimizer=True, overlap_grad_reduce=True,
                     master_as_remainder=True)
    tr = Trainer(cfg, tc, ParallelDims(), device=dev)
    it = synthetic_batch_iterator(cfg.vocab_size, tc.seq_length, 1, dp_rank=0, dp_size=1, pin_memory=True)
    for _ in range(2):
        tr.train_step(it)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        tr.train_step(it)
        torch.cuda.synchronize()
    ka = prof.key_averages()
    rows = sorted([k for k in ka if k.device_time_total > 0 and k.device_type.name == "CUDA"], key=lambda k: -k.device_time_total)
    tot = sum(k.device_time_total for k in rows)
    print(f"total device time {tot/1e3:.1f} ms over {sum(k.count for k in rows)} launches")
    for k in rows[:args.rows]:
        print(f"{k.device_time_total/1e3:9.2f} ms {100*k.device_time_total/tot:5.1f}% n={k.count:5d}  {k.key[:110]}")
    import time
    t0 = time.perf_counter(); tr.train_step(it); torch.cuda.synchronize(); print("wall ms/step", (time.perf_counter()-t0)*1e3)


if __name__ == "__main__":
    main()
