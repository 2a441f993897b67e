"""Distributed optimizer with the peer-memory kernels (gradient reduce-scatter by pull, AdamW + all-gather by push)
against the NCCL path: identical loss curves and parameters on 2 GPUs; and the overlapped parameter all-gather
(``overlap_param_gather``) against the synchronous one, bit for bit."""
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
        from loongforge_b200.data.synthetic import synthetic_batch_iterator
        from loongforge_b200.models.config import TransformerConfig
        from loongforge_b200.ops import _ext
        from loongforge_b200.parallel import state as ps
        from loongforge_b200.runtime.trainer import TrainConfig, Trainer

        def run(peer, overlap_gather=False):
            ps.destroy_model_parallel()
            cfg = TransformerConfig(num_layers=2, hidden_size=512, num_attention_heads=4, num_query_groups=2,
                                    kv_channels=128, ffn_hidden_size=1024, vocab_size=2048)
            tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=256, train_iters=4, lr=1e-3, bf16=True,
                             master_as_remainder=True, peer_optimizer=peer, log_interval=1000,
                             overlap_param_gather=overlap_gather)
            tr = Trainer(cfg, tc, device=torch.device("cuda", rank))
            it = synthetic_batch_iterator(2048, 256, 1, dp_rank=tr.st.dp_rank, dp_size=tr.st.dp_size, seed=5)
            losses = [tr.train_step(it)["lm loss"] for _ in range(4)]
            tr.optimizer.wait_param_gather()  # parameters are read below, outside a forward pass
            torch.cuda.synchronize()
            _ext.check_status()
            return losses, torch.cat([p.detach().float().reshape(-1) for p in tr.models[0].parameters()])

        la, pa = run(False)
        lb, pb = run(True)
        lc, pc = run(False, overlap_gather=True)  # parameter all-gathers queued behind the step, awaited per layer
        # the same trajectory: a stale bucket would show up at once (the first steps move the weights most)
        assert max(abs(a - c) for a, c in zip(la, lc)) < 1e-4 * max(la), f"losses differ: {la} vs {lc}"
        assert float((pa - pc).abs().max()) < 1e-3 * float(pa.abs().max()), "parameters differ after overlapped gathers"
        q.put((rank, "ok", (la, lb, float((pa - pb).abs().max()))))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_optimizer_matches_nccl_path():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for _ in range(2):
            rank, status, payload = q.get(timeout=300)
            assert status == "ok", f"rank {rank}:\n{payload}"
            la, lb, dparam = payload
            assert max(abs(a - b) for a, b in zip(la, lb)) < 2e-2 and dparam < 1e-2, payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
