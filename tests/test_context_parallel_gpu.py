"""Context-parallel attention on GPUs (one process per GPU, NCCL) against the single-GPU flash kernel on the whole
sequence, at a length where a dense score matrix would not be affordable: forward, backward and peak memory."""
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


def _worker(rank, world, port, queue):
    import torch.distributed as dist

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from loongforge_b200.ops import _ext
        from loongforge_b200.ops import functional as OF
        from loongforge_b200.parallel import context_parallel as CP
        from loongforge_b200.parallel import state as ps

        ps.initialize_model_parallel(ps.ParallelDims(cp=world))
        dev = torch.device("cuda", rank)
        T, Hq, Hkv, D = 16384, 8, 2, 128
        torch.manual_seed(3)
        q = torch.randn(T, Hq, D, device=dev).bfloat16()
        k = torch.randn(T, Hkv, D, device=dev).bfloat16()
        v = torch.randn(T, Hkv, D, device=dev).bfloat16()
        do = torch.randn(T, Hq, D, device=dev).bfloat16()
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        ref = OF.attention(qr, kr, vr, causal=True)
        ref.backward(do)
        idx = CP.cp_chunk_indices(T, world, rank, dev)
        out = {}

        def rel(a, b):
            return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()

        for comm in ("allgather", "p2p", "a2a"):
            CP.set_cp_comm_type(comm)
            ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            base = torch.cuda.memory_allocated()
            o = CP.ring_attention(ql, kl, vl, causal=True)
            o.backward(do[idx])
            torch.cuda.synchronize()
            _ext.check_status()
            peak = torch.cuda.max_memory_allocated() - base
            out[comm] = (rel(o, ref[idx]), rel(ql.grad, qr.grad[idx]), rel(kl.grad, kr.grad[idx]),
                         rel(vl.grad, vr.grad[idx]), peak)
        CP.set_cp_comm_type("auto")
        queue.put((rank, "ok", out))
    except Exception:  # noqa: BLE001
        import traceback

        queue.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_matches_single_gpu_kernel(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=240)
            assert status == "ok", f"rank {rank}:\n{payload}"
            for comm, (eo, eq, ek, ev, peak) in payload.items():
                assert eo < 2e-2 and eq < 3e-2 and ek < 3e-2 and ev < 3e-2, (comm, payload[comm])
                # O(T) memory: a dense fp32 score block [8 heads, T/cp, T/cp] alone would be >= 0.5 GB
                assert peak < 400 * 2 ** 20, (comm, peak)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
