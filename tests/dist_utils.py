"""Spawn helper for multi-process CPU (gloo) tests."""
import os
import socket
import sys
import traceback

import torch.multiprocessing as mp


_NEXT_PORT = {"n": 0}


def _free_port() -> int:
    """A port nobody listens on. Test workers running side by side (pytest-xdist) draw from disjoint ranges and never
    hand out the same port twice, so two rendezvous cannot race for one port between probing and binding."""
    w = os.environ.get("PYTEST_XDIST_WORKER", "gw0")
    idx = int(w[2:]) if w[2:].isdigit() else 0
    base = 20000 + (idx % 16) * 2500 + (os.getpid() % 5) * 500
    for _ in range(500):
        port = base + _NEXT_PORT["n"] % 500
        _NEXT_PORT["n"] += 1
        s = socket.socket()
        try:
            s.bind(("127.0.0.1", port))
            return port
        except OSError:
            continue
        finally:
            s.close()
    raise RuntimeError("no free port found")


def _worker(rank, world, port, fn, args, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    import torch
    import torch.distributed as dist

    torch.set_num_threads(2)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        q.put((rank, "ok", out))
    except Exception:  # noqa: BLE001
        q.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def run_distributed(fn, world: int, *args, timeout: float = 600.0):
    """Run ``fn(rank, world, *args)`` on `world` gloo ranks; returns the list of results by rank."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, out = q.get(timeout=timeout)
            if status == "err":
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            results[rank] = out
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
