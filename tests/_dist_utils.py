"""Helpers to run a function on N local ranks (one process per GPU, or CPU ranks on gloo)."""
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, results):
    try:
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(rank)
            kw["device_id"] = torch.device(f"cuda:{rank}")
        dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, **kw)
        out = fn(rank, world, *args)
        results.put((rank, "ok", out))
    except Exception:
        results.put((rank, "error", traceback.format_exc()))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:
            pass


def run_ranks(fn, world, backend="gloo", args=(), timeout=600):
    """Spawn `world` processes running fn(rank, world, *args); return the per-rank results."""
    ctx = mp.get_context("spawn")
    results = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    outs = {}
    while not results.empty():
        rank, status, payload = results.get()
        outs[rank] = (status, payload)
    errors = [f"rank {r}: {v[1]}" for r, v in sorted(outs.items()) if v[0] != "ok"]
    if alive or errors or len(outs) != world:
        raise RuntimeError(f"ranks failed (alive={len(alive)}, reported={len(outs)}/{world}):\n" + "\n".join(errors))
    return [outs[r][1] for r in range(world)]
