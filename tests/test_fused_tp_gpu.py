"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels against plain fp32 products and the NCCL + GEMM path
(needs >= 2 GPUs; spawned as one process per GPU)."""
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


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from loongforge_b200.ops import _ext
        from loongforge_b200.ops import functional as OF
        from loongforge_b200.parallel import fused_tp, mappings as M, state as ps

        ps.initialize_model_parallel(ps.ParallelDims(tp=world))
        g = ps.get_state().group("tp")
        dev = torch.device("cuda", rank)
        errs = {}

        def rel(a, b):
            return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()

        for trial, (T, K, N) in enumerate([(1024, 512, 768), (1024, 512, 768), (2048, 1024, 512), (1024, 512, 768)]):
            torch.manual_seed(100 + trial)  # same weights / full tensors on every rank
            x_full = torch.randn(T, K, device=dev).bfloat16()
            w_full = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
            # ---- all-gather -> GEMM (column parallel: W sharded on N)
            w = w_full.chunk(world, 0)[rank].contiguous().requires_grad_()
            xs = x_full.chunk(world, 0)[rank].contiguous().requires_grad_()
            y = fused_tp.all_gather_linear(xs, w, None)
            gy = torch.randn_like(y)
            y.backward(gy)
            w2 = w.detach().clone().requires_grad_()
            xs2 = xs.detach().clone().requires_grad_()
            yr = OF.linear(M.gather_from_sequence_parallel_region(xs2, g, True), w2)
            yr.backward(gy)
            errs[f"ag{trial}_y"] = rel(y, yr)
            # also against a plain fp32 product of the full operands (not only against the library path)
            y32 = x_full.float() @ w_full.float().t()
            errs[f"ag{trial}_y_fp32"] = rel(y, y32.chunk(world, 1)[rank])
            errs[f"ag{trial}_dw_fp32"] = rel(w.grad, gy.float().t() @ x_full.float())
            gy_all = [torch.empty_like(gy) for _ in range(world)]
            dist.all_gather(gy_all, gy)
            dx32 = sum(gy_all[r].float() @ w_full.chunk(world, 0)[r].float() for r in range(world))
            errs[f"ag{trial}_dx_fp32"] = rel(xs.grad, dx32.chunk(world, 0)[rank])
            errs[f"ag{trial}_dx"] = rel(xs.grad, xs2.grad)
            errs[f"ag{trial}_dw"] = rel(w.grad, w2.grad)
            # ---- GEMM -> reduce-scatter (row parallel: W sharded on K), with residual
            wr = w_full.chunk(world, 1)[rank].contiguous().requires_grad_()
            xr = x_full.chunk(world, 1)[rank].contiguous().requires_grad_()
            res = torch.randn(T // world, N, device=dev).bfloat16().requires_grad_()
            z = fused_tp.linear_reduce_scatter(xr, wr, res)
            gz = torch.randn_like(z)
            z.backward(gz)
            wr2 = wr.detach().clone().requires_grad_()
            xr2 = xr.detach().clone().requires_grad_()
            zr = M.reduce_scatter_to_sequence_parallel_region(OF.linear(xr2, wr2), g) + res.detach()
            zr.backward(gz)
            errs[f"rs{trial}_z"] = rel(z, zr)
            z32 = (x_full.float() @ w_full.float().t()).chunk(world, 0)[rank] + res.detach().float()
            errs[f"rs{trial}_z_fp32"] = rel(z, z32)
            gz_all = [torch.empty_like(gz) for _ in range(world)]
            dist.all_gather(gz_all, gz)
            gz_full = torch.cat(gz_all).float()
            errs[f"rs{trial}_dx_fp32"] = rel(xr.grad, gz_full @ w_full.chunk(world, 1)[rank].float())
            errs[f"rs{trial}_dw_fp32"] = rel(wr.grad, gz_full.t() @ x_full.chunk(world, 1)[rank].float())
            errs[f"rs{trial}_dx"] = rel(xr.grad, xr2.grad)
            errs[f"rs{trial}_dw"] = rel(wr.grad, wr2.grad)
            errs[f"rs{trial}_dres"] = rel(res.grad, gz)
        torch.cuda.synchronize()
        _ext.check_status()
        dist.barrier()
        q.put((rank, "ok", errs))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            import torch.distributed as dist

            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_kernels_match_nccl_reference():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=300)
            assert status == "ok", f"rank {rank}:\n{payload}"
            out[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, errs in out.items():
        for k, v in errs.items():
            assert v < 2e-2, f"rank {rank} {k}: rel err {v}"
