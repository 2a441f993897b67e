"""MoE layer with the NVLink peer-memory dispatcher against the NCCL all-to-all dispatcher
(1 GPU: expert parallel size 1; 2 GPUs: expert parallel size 2, one process per GPU)."""
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


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _compare_layers(dev, ep, seed_shift=0, steps=3):
    """Builds the same MoE layer twice (alltoall / peer), runs a few forward+backward passes on
    different tokens (exercising buffer reuse) and returns relative errors."""
    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.models.moe import MoELayer

    kw = dict(num_layers=2, hidden_size=256, num_attention_heads=2, num_query_groups=2, kv_channels=128,
              ffn_hidden_size=512, vocab_size=1024, num_moe_experts=8, moe_router_topk=2, moe_ffn_hidden_size=256,
              moe_aux_loss_coeff=0.0, params_dtype=torch.bfloat16)
    ref = MoELayer(TransformerConfig(**kw), "decoder.layers.0.mlp", 0, device=dev)
    # a capacity factor this small forces the receive buffers to be re-allocated when routing is skewed
    peer = MoELayer(TransformerConfig(moe_token_dispatcher_type="peer", moe_peer_capacity_factor=0.55, **kw),
                    "decoder.layers.0.mlp", 0, device=dev)
    peer.load_state_dict(ref.state_dict())
    errs = {}
    for step in range(steps):
        torch.manual_seed(7 + step + seed_shift)
        T = 384 + 128 * step
        x = torch.randn(T, 256, device=dev).bfloat16()
        xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
        gy = torch.randn(T, 256, device=dev).bfloat16()
        ya = ref(xa)
        ya.backward(gy)
        yb = peer(xb)
        yb.backward(gy)
        errs[f"y{step}"] = _rel(yb, ya)
        errs[f"dx{step}"] = _rel(xb.grad, xa.grad)
    for (n, pa), (_, pb) in zip(ref.named_parameters(), peer.named_parameters()):
        errs["d_" + n] = _rel(pb.grad, pa.grad)
    return errs


def test_peer_dispatcher_single_gpu():
    from loongforge_b200.ops import _ext
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    errs = _compare_layers(torch.device("cuda", 0), 1)
    _ext.check_status()
    for k, v in errs.items():
        assert v < 3e-2, f"{k}: {v}"


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from loongforge_b200.ops import _ext
        from loongforge_b200.parallel import state as ps

        ps.initialize_model_parallel(ps.ParallelDims(ep=world))
        errs = _compare_layers(torch.device("cuda", rank), world, seed_shift=100 * rank)
        torch.cuda.synchronize()
        _ext.check_status()
        dist.barrier()
        q.put((rank, "ok", errs))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_dispatcher_expert_parallel_two_gpus():
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
            assert v < 3e-2, f"rank {rank} {k}: rel err {v}"
