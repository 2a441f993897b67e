"""EMA, sparse upcycling, profiler / inspector hooks, scalar writers, asynchronous + local checkpoints, retention."""
import json
import os

import torch

from loongforge_b200.parallel import state as ps


def test_ema_tracks_and_swaps():
    from loongforge_b200.runtime.ema import ModelEMA

    m = torch.nn.Linear(3, 3)
    ema = ModelEMA(m.named_parameters(), decay=0.5, warmup=False)
    w0 = m.weight.detach().clone()
    with torch.no_grad():
        m.weight.add_(2.0)
    ema.update()
    assert torch.allclose(ema.shadow["weight"], w0 + 1.0)
    with ema.swapped_in():
        assert torch.allclose(m.weight, w0 + 1.0)
    assert torch.allclose(m.weight, w0 + 2.0)
    e2 = ModelEMA(m.named_parameters(), decay=0.9)
    e2.load_state_dict(ema.state_dict())
    assert torch.equal(e2.shadow["weight"], ema.shadow["weight"]) and e2.updates == 1


def test_upcycled_moe_reproduces_dense_output():
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.runtime.upcycling import upcycle_state_dict

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    base = dict(vocab_size=256, num_layers=1)
    dense = build_model(get_model_config("tiny-llama", **base))
    cfg = get_model_config("tiny-llama", num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=688 // 2,
                           moe_router_pre_softmax=False, moe_aux_loss_coeff=0.0, **base)
    moe = build_model(cfg)
    sd = upcycle_state_dict(dense.state_dict(), 4, granularity=2, router_std=0.0)
    missing, unexpected = moe.load_state_dict(sd, strict=False)
    assert not unexpected and not [k for k in missing if "_extra_state" not in k], (missing, unexpected)
    # a zero router ties all experts; make the top-2 pick one expert of each slice with weights 1/2 each
    with torch.no_grad():
        moe.decoder.layers[0].mlp.router.weight.zero_()
    tokens, pos = torch.randint(0, 256, (16,)), torch.arange(16)
    a, b = dense(tokens, pos), moe(tokens, pos)
    assert torch.allclose(a, b, atol=2e-4), (a - b).abs().max()


def test_profiler_inspector_and_writers(tmp_path):
    from loongforge_b200.runtime import metrics_writers as W, profiling as P

    prof = P.StepProfiler(str(tmp_path), 1, 3, ranks=[0], rank=0, profile_memory=False)
    for it in range(5):
        torch.randn(64, 64) @ torch.randn(64, 64)
        prof.step(it)
    assert prof.trace_path and os.path.getsize(prof.trace_path) > 0
    assert P.detail_iteration(20, 10) and not P.detail_iteration(21, 10) and not P.detail_iteration(5, None)
    with P.nvtx_range("x"):
        pass
    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU(), torch.nn.Linear(4, 2))
    insp = P.TensorInspector(m, ["0", "2"], str(tmp_path / "tensors.jsonl"))
    m(torch.randn(3, 4)).sum().backward()
    insp.step()
    recs = [json.loads(x) for x in open(tmp_path / "tensors.jsonl")]
    assert {(r["module"], r["kind"]) for r in recs} == {("0", "fwd"), ("2", "fwd"), ("0", "bwd"), ("2", "bwd")}
    insp.remove()
    w = W.ScalarWriter(str(tmp_path / "tb"), tensorboard=True)
    w.add_scalars({"lm loss": 2.5, "lr": 1e-4}, 3)
    w.close()
    assert json.loads(open(tmp_path / "tb" / "scalars.jsonl").readline())["lm loss"] == 2.5
    pl = W.ProgressLog(str(tmp_path), 8)
    pl.start(0.0, "job1")
    pl.checkpoint(10, 1000, 8e12)
    assert "Saved checkpoint" in open(tmp_path / "progress.txt").read()
    assert W.EnergyMonitor().lap() >= 0.0
    txt = W.dump_first_batch({"tokens": torch.tensor([5, 6, 7]), "loss_mask": torch.tensor([0, 1, 1])})
    assert "5 [6] [7]" in txt


def test_async_local_checkpoints_and_retention(tmp_path):
    from loongforge_b200.ckpt import async_save as A

    saver = A.AsyncSaver()
    state = {"w": torch.arange(4.0), "nested": {"step": 3, "t": [torch.ones(2)]}}
    done = []
    saver.save(str(tmp_path / "iter_0000004" / "x.pt"), state, on_done=lambda: done.append(1))
    state["w"].zero_()  # the staged copy is what gets written
    saver.wait()
    back = torch.load(tmp_path / "iter_0000004" / "x.pt", weights_only=False)
    assert done == [1] and torch.equal(back["w"], torch.arange(4.0)) and back["nested"]["step"] == 3
    for i in (2, 6, 8, 10):
        os.makedirs(tmp_path / f"iter_{i:07d}", exist_ok=True)
    assert A.apply_retention(str(tmp_path), keep_last=1, retain_interval=4) == [2, 6]
    assert A.list_iterations(str(tmp_path)) == [4, 8, 10]
    loc = A.LocalCheckpointManager(str(tmp_path / "local"), rank=1)
    loc.save(11, {"a": torch.ones(1)})
    loc.save(12, {"a": torch.full((1,), 2.0)})
    assert A.list_iterations(str(tmp_path / "local")) == [12]
    assert loc.find_latest(10) == 12 and loc.find_latest(12) is None and float(loc.load(12)["a"]) == 2.0
    A.save_dataloader_state(str(tmp_path), 3, {"consumed": 77})
    assert A.load_dataloader_state(str(tmp_path), 3) == {"consumed": 77} and A.load_dataloader_state(str(tmp_path), 4) is None
    ex = A.ExitDecider(exit_interval=5)
    assert ex.should_exit(10) == "interval" and ex.should_exit(11) is None
    ex._on_signal(15, None)
    assert ex.should_exit(11) == "signal"


def test_cli_hooks_end_to_end(tmp_path):
    """Flags -> hooks: EMA checkpoint, scalar file, profiler trace, tensor log, exit-interval checkpoint."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "run"
    cmd = [sys.executable, "-m", "loongforge_b200.train", "--model-name", "tiny-llama", "--seq-length", "64",
           "--micro-batch-size", "2", "--global-batch-size", "4", "--train-iters", "6", "--lr", "1e-3", "--ema-decay", "0.99",
           "--tensorboard-dir", str(out), "--profile", "--profile-step-start", "2", "--profile-step-end", "4",
           "--enable-log-tensor", "--log-tensor-name-pattern", "decoder.layers.0.mlp", "--manual-gc",
           "--exit-interval", "5", "--save", str(out / "ck")]
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert p.returncode == 0, p.stderr[-2000:]
    assert "iteration        5/" in p.stdout and "iteration        6/" not in p.stdout  # left at the exit interval
    assert (out / "ck" / "iter_0000005").is_dir() and (out / "ck" / "save_ema" / "iter_0000005").is_dir()
    assert len(open(out / "scalars.jsonl").readlines()) == 5
    assert (out / "trace_rank0_it2-4.json").is_file()
    recs = [json.loads(x) for x in open(out / "tensors_rank0.jsonl")]
    assert recs and all(r["module"].endswith("decoder.layers.0.mlp") for r in recs)


def _offload_traj(rank, world, offload, fraction=1.0):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-llama")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=4, lr=1e-3, clip_grad=0.5,
                     weight_decay=0.1, log_interval=1000, optimizer_cpu_offload=offload,
                     optimizer_offload_fraction=fraction, ddp_bucket_size=20000)
    tr = Trainer(cfg, tc)
    st = tr.st
    it = synthetic_batch_iterator(cfg.vocab_size, 64, 1, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=11,
                                  pin_memory=False)
    out = [tr.train_step(it) for _ in range(4)]
    shards = tr.optimizer.shards
    if offload and fraction >= 1.0:
        assert all(sh.offload and sh.exp_avg.device.type == "cpu" for sh in shards)
    elif offload:
        total = sum(sh.end - sh.start for sh in shards)
        on_host = sum(sh.end - sh.start for sh in shards if sh.offload)
        assert len(shards) > 2 and 0 < on_host < total and on_host >= fraction * total - max(
            sh.end - sh.start for sh in shards), (on_host, total)
    return [(m["lm loss"], m["grad_norm"]) for m in out]


def test_optimizer_cpu_offload_matches_device_optimizer():
    """Sharded optimizer over 2 data-parallel ranks: the host AdamW path follows the on-device trajectory."""
    from dist_utils import run_distributed

    a = run_distributed(_offload_traj, 2, False)[0]
    b = run_distributed(_offload_traj, 2, True)[0]
    for (l0, g0), (l1, g1) in zip(a, b):
        assert abs(l0 - l1) < 1e-5 * max(1, abs(l0)) and abs(g0 - g1) < 1e-4 * max(1, abs(g0)), (a, b)


def test_optimizer_offload_fraction_keeps_part_of_the_state_on_the_device():
    from dist_utils import run_distributed

    a = run_distributed(_offload_traj, 2, False)[0]
    b = run_distributed(_offload_traj, 2, True, 0.5)[0]
    for (l0, g0), (l1, g1) in zip(a, b):
        assert abs(l0 - l1) < 1e-5 * max(1, abs(l0)) and abs(g0 - g1) < 1e-4 * max(1, abs(g0)), (a, b)


def test_sgd_with_momentum_follows_the_torch_update_rule():
    """--optimizer sgd on the flat-buffer optimizer: with the gradients read back from the gradient buffer, the
    parameters follow torch.optim.SGD (momentum, weight decay) step by step."""
    import torch

    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    ps.destroy_model_parallel()
    cfg = get_model_config("tiny-llama")
    tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=3, lr=0.05, min_lr=0.05,
                     lr_decay_style="constant", clip_grad=0.0, weight_decay=0.01, log_interval=1000, optimizer="sgd",
                     sgd_momentum=0.8)
    tr = Trainer(cfg, tc)
    named = dict(tr.models[0].module.named_parameters())
    ref = {n: torch.nn.Parameter(p.detach().clone().float()) for n, p in named.items()}
    groups = [{"params": [ref[n] for n, p in named.items() if p.dim() > 1], "weight_decay": 0.01},
              {"params": [ref[n] for n, p in named.items() if p.dim() <= 1], "weight_decay": 0.0}]
    opt = torch.optim.SGD(groups, lr=0.05, momentum=0.8)
    it = synthetic_batch_iterator(cfg.vocab_size, 32, 2, seed=3, pin_memory=False)
    for step in range(3):
        tr.train_step(it)
        for n, p in named.items():   # the gradient buffer still holds this step's reduced gradients
            ref[n].grad = p.main_grad.detach().clone().float()
        opt.step()
        worst = max(float((ref[n].detach() - p.detach().float()).abs().max()) for n, p in named.items())
        assert worst < 1e-5, (step, worst)
    ps.destroy_model_parallel()


def _fsdp_traj(rank, world, use_fsdp, tmp):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig
    from loongforge_b200.runtime.trainer_builder import build_model_trainer

    def make():
        cfg = get_model_config("tiny-llama")
        tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=6, lr=1e-3, clip_grad=0.5,
                         weight_decay=0.1, log_interval=1000, use_fsdp=use_fsdp)
        return build_model_trainer("llama", "pretrain", model_cfg=cfg, train_cfg=tc, dims=None), cfg

    tr, cfg = make()
    st = tr.st
    data = lambda start=0: synthetic_batch_iterator(cfg.vocab_size, 64, 1, dp_rank=st.dp_rank, dp_size=st.dp_size,  # noqa: E731
                                                    seed=11, pin_memory=False, start_sample=start)
    it = data()
    out = [tr.train_step(it) for _ in range(3)]
    traj = [(m["lm loss"], m["grad_norm"]) for m in out]
    if not use_fsdp:
        return traj, None
    assert type(tr).__name__ == "FSDPTrainer"
    w = tr.models[0].module.decoder.layers[0].mlp.linear_fc1.weight
    assert w.to_local().shape[0] * world == w.shape[0], "parameters are sharded over the data-parallel ranks"
    tr.save_checkpoint(tmp)
    cont = tr.train_step(it)
    ps.destroy_model_parallel()
    tr2, _ = make()
    assert tr2.load_checkpoint(tmp) == 3
    again = tr2.train_step(data(tr2.consumed_samples))
    return traj, (cont["lm loss"], again["lm loss"], cont["grad_norm"], again["grad_norm"])


def test_fsdp_trainer_matches_ddp_trainer_and_resumes(tmp_path):
    from dist_utils import run_distributed

    a = run_distributed(_fsdp_traj, 2, False, str(tmp_path))[0][0]
    b, resume = run_distributed(_fsdp_traj, 2, True, str(tmp_path))[0]
    for (l0, g0), (l1, g1) in zip(a, b):
        assert abs(l0 - l1) < 1e-4 * max(1, abs(l0)) and abs(g0 - g1) < 1e-3 * max(1, abs(g0)), (a, b)
    c, again, gc, ga = resume
    assert abs(c - again) < 1e-6 and abs(gc - ga) < 1e-5, resume


def test_fp8_blockwise_training_follows_the_full_precision_run(tmp_path):
    """FP8 forward / input-gradient GEMMs (emulated bit-exactly on CPU) in every supported linear layer: the loss
    follows the fp32 run closely, the policy file can keep kinds in bf16, and unsupported modules stay in bf16."""
    import json

    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    def run(fp8, policy=None):
        ps.destroy_model_parallel()
        cfg = get_model_config("tiny-llama", fp8=fp8, ffn_hidden_size=512)
        tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=64, train_iters=6, lr=1e-3,
                         log_interval=1000, fp8_policy_file=policy)
        tr = Trainer(cfg, tc)
        it = synthetic_batch_iterator(cfg.vocab_size, 64, 2, seed=2, pin_memory=False)
        return [tr.train_step(it)["lm loss"] for _ in range(6)], tr.fp8_decisions

    ref, none = run(None)
    got, dec = run("blockwise")
    assert none == {} and dec
    assert all(v == "fp8" for k, v in dec.items() if k.endswith(("linear_qkv", "linear_fc1", "linear_fc2")))
    assert dec["output_layer"] == "bf16"
    assert got != ref, "the FP8 path must actually change the arithmetic"
    assert all(abs(a - b) < 5e-3 * abs(a) for a, b in zip(ref, got)), (ref, got)
    pol = tmp_path / "policy.json"
    pol.write_text(json.dumps({"default": "bf16", "rules": [{"kind": "linear_fc1", "precision": "fp8"}]}))
    _, dec2 = run("blockwise", str(pol))
    assert {v for k, v in dec2.items() if k.endswith("linear_fc1")} == {"fp8"}
    assert {v for k, v in dec2.items() if not k.endswith("linear_fc1")} == {"bf16"}


def _balance_run(rank, world, balance):
    import torch

    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-llama")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=8, seq_length=256, train_iters=2, lr=1e-3, clip_grad=1.0,
                     log_interval=1000, dp_balance=balance)
    tr = Trainer(cfg, tc)
    # rank 0 always draws the long sequences, rank 1 the short ones: the worst case for lock-step data parallelism
    lens = [256, 224, 192, 160] if tr.st.dp_rank == 0 else [32, 48, 64, 16]

    def it():
        g = torch.Generator().manual_seed(100 + tr.st.dp_rank)
        while True:
            for T in lens:
                tok = torch.randint(0, cfg.vocab_size, (1, T + 1), generator=g)
                yield {"tokens": tok[:, :-1], "labels": tok[:, 1:], "loss_mask": torch.ones(1, T),
                       "position_ids": torch.arange(T)[None], "tag": (tr.st.dp_rank, T)}

    seen = []
    orig = tr.get_batch
    tr.get_batch = lambda di: (lambda b: (seen.append(b["tag"]), b)[1])(orig(di))
    out = [tr.train_step(it_) for it_ in [it()] * 1 for _ in range(2)]
    w = tr.__dict__.get("_balanced_iterators")
    imb = next(iter(w.values())).last_imbalance if w else None
    return [(m["lm loss"], m["grad_norm"]) for m in out], seen, imb


def test_dp_balance_moves_microbatches_without_changing_the_step():
    from dist_utils import run_distributed

    plain = run_distributed(_balance_run, 2, False)
    bal = run_distributed(_balance_run, 2, True)
    for (l0, g0), (l1, g1) in zip(plain[0][0], bal[0][0]):
        assert abs(l0 - l1) < 1e-5 * abs(l0) and abs(g0 - g1) < 1e-4 * max(1, g0), (plain[0][0], bal[0][0])
    (_, seen0, imb0), (_, seen1, imb1) = bal
    assert imb0 == imb1 and imb0[1] < imb0[0] and imb0[1] < 1.2, imb0
    assert len(seen0) == len(seen1) == 8, "every rank keeps its micro-batch count"
    assert {r for r, _ in seen0} == {0, 1}, "rank 0 now also processes micro-batches that rank 1 loaded"
    assert sorted(seen0[:4] + seen1[:4]) == sorted(plain[0][1][:4] + plain[1][1][:4]), "the step's batch set is unchanged"


def _resilient(rank, world, kind, rate):
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = get_model_config("tiny-llama")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=6, lr=1e-3, log_interval=1000,
                     rerun_mode="validate_results", error_injection_rate=rate, error_injection_type=kind, seed=5,
                     iterations_to_skip=[2], check_weight_hash_interval=1)
    tr = Trainer(cfg, tc)
    st = tr.st
    pulled = []

    def it():
        for b in synthetic_batch_iterator(cfg.vocab_size, 64, 1, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=3,
                                          pin_memory=False):
            pulled.append(1)
            yield b

    hist = tr.train(it())
    return [m["skipped"] for m in hist], tr.rerun.stats, tr.exit_requested, tr.iteration, len(pulled)


def test_rerun_machine_error_injection_and_iteration_skipping():
    from dist_utils import run_distributed

    # transient faults: every corrupted loss is replayed once, comes back clean, and the step is applied
    skipped, stats, exit_reason, it, pulled = run_distributed(_resilient, 2, "transient_error", 2)[0]
    assert exit_reason is None and it == 6 and sum(skipped) == 0 and stats["nan"] >= 1 and stats["transient"] == stats["nan"]
    assert len(skipped) == 5 and pulled == 6 * 2, "iteration 2 trained nothing but consumed its two micro-batches"
    # a persistent fault reproduces on replay: no update, checkpoint-and-exit requested, the loop stops
    skipped, stats, exit_reason, it, _ = run_distributed(_resilient, 2, "persistent_error", 1)[0]
    assert exit_reason and "persistent" in exit_reason and stats["persistent"] == 1 and skipped == [1] and it == 1


def test_straggler_and_heartbeat_hooks():
    import types

    import torch.distributed as dist

    from loongforge_b200.runtime import hooks as H

    tr = types.SimpleNamespace(tcfg=types.SimpleNamespace(log_interval=2), iteration=0)
    lines = []
    sh = H.StragglerHook(tr, threshold=1.3, sink=lines.append)
    for i in range(4):
        tr.iteration = i + 1
        sh.on_step_end(tr, {}, 100.0)
    assert len(sh.reports) == 2 and sh.reports[0]["stragglers"] == [] and not lines
    store = dist.HashStore()
    a, b = H.HeartbeatHook(store, 0, 2, timeout_s=5.0), H.HeartbeatHook(store, 1, 2, timeout_s=5.0)
    assert a.on_step_end(tr, {}, 1.0) is None and b.on_step_end(tr, {}, 1.0) is None
    # rank 1 stops beating; rank 0 keeps going and notices once the timeout has passed (time is injected, not slept)
    a.hb.beat()
    assert a.hb.dead_ranks(now=1000.0) == []          # observes rank 1's first beat
    assert a.hb.dead_ranks(now=1004.0) == []          # unchanged, but within the timeout
    assert a.hb.dead_ranks(now=1006.0) == [1]         # unchanged for longer than the timeout
    b.hb.beat()
    assert a.hb.dead_ranks(now=1007.0) == []


def _leaver(rank, world):
    """Rank 1 leaves between steps (no collective in flight); rank 0 learns of it from the store, not from a hang."""
    import time

    import torch.distributed as dist

    from loongforge_b200.runtime.resilience import Heartbeat

    hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, timeout_s=1.0)
    dist.barrier()
    for step in range(40):
        hb.beat()
        if rank == 1 and step == 2:
            return "left"
        dead = hb.dead_ranks()
        if dead:
            return ("detected", dead, step)
        time.sleep(0.2)
    return "never noticed"


def test_rank_that_leaves_is_detected_through_the_store():
    from dist_utils import run_distributed

    r0, r1 = run_distributed(_leaver, 2)
    assert r1 == "left" and r0[0] == "detected" and r0[1] == [1] and r0[2] > 2


def test_cli_start_state_precedence_and_hf_export(tmp_path):
    """Run A trains and writes Hugging Face weights; run B starts from those HF weights; run C fine-tunes from A's
    checkpoint given as --pretrained-checkpoint (iteration restarts at 0); run D resumes A at a chosen step."""
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root)
    base = [sys.executable, "-m", "loongforge_b200.train", "--model-name", "tiny-llama", "--seq-length", "64",
            "--micro-batch-size", "2", "--global-batch-size", "2", "--lr", "1e-3", "--log-interval", "1"]

    def run(extra):
        p = subprocess.run(base + extra, cwd=root, capture_output=True, text=True, timeout=600, env=env)
        assert p.returncode == 0, p.stderr[-2000:]
        return [(int(m.group(1)), float(m.group(2))) for m in
                re.finditer(r"iteration\s+(\d+)/.*?lm loss: ([0-9.E+-]+)", p.stdout)]

    a = run(["--train-iters", "4", "--save", str(tmp_path / "a"), "--save-interval", "2", "--save-hf"])
    hf = tmp_path / "a" / "release_hf_weights"
    assert (hf / "config.json").is_file() and any(f.suffix == ".safetensors" for f in hf.iterdir())
    assert [i for i, _ in a] == [1, 2, 3, 4]
    fresh = run(["--train-iters", "1"])
    # B: --load pointing at a Hugging Face directory -> online conversion, iteration 0, trained weights (lower loss)
    b = run(["--train-iters", "1", "--load", str(hf)])
    assert b[0][0] == 1 and b[0][1] < fresh[0][1] - 1e-3
    # C: --pretrained-checkpoint -> weights only, the schedule starts over
    c = run(["--train-iters", "1", "--pretrained-checkpoint", str(tmp_path / "a")])
    assert c[0][0] == 1 and abs(c[0][1] - b[0][1]) < 1e-3 * b[0][1]
    # D: resume at --ckpt-step 2 -> continues with iteration 3 and reproduces run A's iteration 3
    d = run(["--train-iters", "3", "--load", str(tmp_path / "a"), "--ckpt-step", "2"])
    assert d[0][0] == 3 and abs(d[0][1] - a[2][1]) < 1e-5 * a[2][1]


def test_batch_size_rampup_and_sample_based_flags(monkeypatch):
    from loongforge_b200.config.arguments import parse_args
    from loongforge_b200.config.build import build_configs
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.runtime.trainer import Trainer

    monkeypatch.setenv("WORLD_SIZE", "1")
    args, ov = parse_args(["--model-name", "tiny-llama", "--seq-length", "32", "--micro-batch-size", "1",
                           "--global-batch-size", "4", "--train-samples", "40", "--rampup-batch-size", "2", "2", "8",
                           "--lr", "1e-3", "--lr-warmup-fraction", "0.2", "--num-layers-per-virtual-pipeline-stage", "1",
                           "--accumulate-allreduce-grads-in-fp32", "--attention-dropout", "0.0", "--mock-data"])
    cfg, tc, dims, _ = build_configs(args, ov)
    assert tc.train_iters == 10 and tc.lr_warmup_iters == 2 and tc.rampup_batch_size == [2, 2, 8]
    assert tc.grad_reduce_in_fp32 and dims.vpp == 2 and cfg.attention_dropout == 0.0
    dims.vpp = None
    tr = Trainer(cfg, tc, dims)
    it = synthetic_batch_iterator(cfg.vocab_size, 32, 1, pin_memory=False)
    sizes = []
    for _ in range(6):
        tr.train_step(it)
        sizes.append(tr.mb_calc.current_gbs)
    assert sizes == [2, 2, 2, 2, 4, 4] and tr.consumed_samples == 16
    assert "global batch size:     4" in tr.format_log({"lm loss": 1.0, "grad_norm": 1.0}, 10.0)


def test_timing_log_level_reports_phase_times():
    from loongforge_b200.data.synthetic import synthetic_batch_iterator
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    ps.destroy_model_parallel()
    cfg = get_model_config("tiny-llama")
    seen = {}
    for level in (0, 2):
        tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=32, train_iters=2, lr=1e-3, log_interval=2,
                         timing_log_level=level, log_timers_to_tensorboard=True)
        tr = Trainer(cfg, tc)
        lines = []
        hist = tr.train(synthetic_batch_iterator(cfg.vocab_size, 32, 1, seed=1, pin_memory=False), on_log=lines.append)
        seen[level] = ("\n".join(lines), hist[-1])
        ps.destroy_model_parallel()
    assert "forward-backward" not in seen[0][0] and not any(k.startswith("timers/") for k in seen[0][1])
    text, last = seen[2]
    for name in ("forward-backward", "optimizer", "partial-grads-all-reduce", "loss-reduce"):
        assert name in text, text
    assert last["timers/forward-backward-ms"] > 0 and last["timers/optimizer-ms"] > 0


def _dp_balance_fit(rank, world):
    import numpy as np

    from loongforge_b200.data.dp_balance import CostModel, fit_cost_model_across_ranks

    m = CostModel()
    rng = np.random.RandomState(rank)
    for _ in range(4):  # each rank alone has too few distinct observations for a 3-parameter fit to be trusted
        ls = [int(x) for x in rng.randint(50, 400, size=3)]
        m.observe(ls, sum(2e-5 * s * s + 3e-3 * s + 0.5 for s in ls))
    return [float(c) for c in fit_cost_model_across_ranks(m)], len(m.obs)


def test_dp_balance_warmup_fit_pools_observations_of_all_ranks():
    from dist_utils import run_distributed

    res = run_distributed(_dp_balance_fit, 2)
    (c0, n0), (c1, n1) = res
    assert n0 == n1 == 8 and c0 == c1  # same pooled observations -> same plan on every rank
    assert abs(c0[0] - 2e-5) < 1e-7 and abs(c0[1] - 3e-3) < 1e-4 and abs(c0[2] - 0.5) < 5e-2


def test_cli_separate_train_and_validation_data(tmp_path):
    """--train-data-path / --valid-data-path for pretraining (.bin / .idx prefixes) and for SFT (named layouts), with
    periodic evaluation on the validation stream."""
    import json
    import subprocess
    import sys
    from tools.data_preprocess import preprocess_pretrain_data as pp

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for name, n in (("train", 60), ("valid", 12)):
        (tmp_path / f"{name}.jsonl").write_text("\n".join(json.dumps({"text": f"{name} document {i} " + "word " * 40}) for i in range(n)))
        pp.main(["--input", str(tmp_path / f"{name}.jsonl"), "--output-prefix", str(tmp_path / name), "--append-eod"])
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root)
    base = [sys.executable, "-m", "loongforge_b200.train", "--model-name", "tiny-llama", "--seq-length", "64", "--micro-batch-size", "1",
            "--global-batch-size", "2", "--train-iters", "4", "--lr", "1e-3", "--log-interval", "1", "--eval-interval", "2", "--eval-iters", "2"]
    p = subprocess.run(base + ["--train-data-path", str(tmp_path / "train_text_document"), "--valid-data-path", str(tmp_path / "valid_text_document"),
                               "--tokenizer-type", "NullTokenizer", "--vocab-size", "512"], cwd=root, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert p.stdout.count("validation loss at iteration") >= 2 or p.stdout.count("validation") >= 2, p.stdout[-1500:]
    (tmp_path / "sft_train.jsonl").write_text("\n".join(json.dumps({"instruction": f"say {i}", "input": "", "output": f"{i} " * 5}) for i in range(16)))
    (tmp_path / "sft_valid.jsonl").write_text("\n".join(json.dumps({"instruction": f"tell {i}", "input": "", "output": f"{i}"}) for i in range(6)))
    q = subprocess.run(base + ["--training-phase", "sft", "--sft-dataset", "alpaca", "--train-data-path", str(tmp_path / "sft_train.jsonl"),
                               "--valid-data-path", str(tmp_path / "sft_valid.jsonl"), "--chat-template", "chatml", "--packing-sft-data",
                               "--tokenizer-type", "NullTokenizer", "--vocab-size", "512"], cwd=root, capture_output=True, text=True, timeout=600, env=env)
    assert q.returncode == 0, q.stdout[-1500:] + q.stderr[-3000:]
    assert q.stdout.count("validation") >= 2, q.stdout[-1500:]
