"""Layouts that so far ran on gloo ranks only, on GPUs over NCCL (one process per GPU): pipeline parallelism (1F1B and
interleaved 1F1B), and the MoE all-to-all overlap schedule with both dispatchers. Each layout must reproduce the
single-GPU trajectory of the same model, data and seed within bf16 tolerance."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, queue, model_name, dims_kw, train_kw, cfg_kw):
    import torch.distributed as dist

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from loongforge_b200.data.synthetic import synthetic_batch_iterator
        from loongforge_b200.models.registry import get_model_config
        from loongforge_b200.ops import _ext
        from loongforge_b200.parallel.state import ParallelDims
        from loongforge_b200.runtime.trainer import TrainConfig, Trainer

        cfg = get_model_config(model_name, **cfg_kw)
        tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=256, train_iters=3, lr=1e-3, clip_grad=1.0,
                         bf16=True, log_interval=1000, **train_kw)
        tr = Trainer(cfg, tc, ParallelDims(**dims_kw), device=dev)
        st = tr.st
        it = synthetic_batch_iterator(cfg.vocab_size, 256, 1, dp_rank=st.dp_rank, dp_size=st.dp_size, seed=3,
                                      pin_memory=True)
        out = []
        for _ in range(3):
            m = tr.train_step(it)
            out.append((m.get("lm loss"), m["grad_norm"]))
        torch.cuda.synchronize()
        _ext.check_status()
        queue.put((rank, "ok", out))
    except Exception:  # noqa: BLE001
        import traceback

        queue.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _launch(world, model_name, dims_kw, train_kw=None, cfg_kw=None):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, queue, model_name, dict(dims_kw), dict(train_kw or {}),
                                               dict(cfg_kw or {}))) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, status, payload = queue.get(timeout=240)
            assert status == "ok", f"rank {rank}:\n{payload}"
            res[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return res


def _close(ref, got, tol):
    for (l0, g0), (l1, g1) in zip(ref, got):
        if l1 is not None:
            assert abs(l0 - l1) < tol * max(1.0, abs(l0)), (ref, got)
        assert abs(g0 - g1) < 5 * tol * max(1.0, abs(g0)), (ref, got)


@pytest.mark.parametrize("dims", [{"pp": 2}, {"pp": 2, "vpp": 2}])
def test_pipeline_parallel_on_nccl_matches_single_gpu(dims):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ck = {"num_layers": 4}
    ref = _launch(1, "tiny-llama", {}, {}, ck)[0]
    got = _launch(2, "tiny-llama", dims, {}, ck)
    _close(ref, got[1], 2e-2)  # the last stage reports the loss


@pytest.mark.parametrize("dispatcher", ["alltoall", "peer"])
def test_a2a_overlap_on_gpus_matches_plain_step(dispatcher):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ck = {"moe_token_dispatcher_type": dispatcher}
    plain = _launch(2, "tiny-qwen3-moe", {"ep": 2}, {}, ck)
    over = _launch(2, "tiny-qwen3-moe", {"ep": 2}, {"overlap_moe_expert_parallel_comm": True}, ck)
    for r in (0, 1):
        _close(plain[r], over[r], 5e-3)


def test_a2a_overlap_single_gpu_matches_plain_step():
    plain = _launch(1, "tiny-qwen3-moe", {})[0]
    over = _launch(1, "tiny-qwen3-moe", {}, {"overlap_moe_expert_parallel_comm": True})[0]
    _close(plain, over, 5e-3)
