"""Run a function as `world` ranks in child processes (127.0.0.1 rendezvous) and collect its results: Gloo on CPU
by default, NCCL with one GPU per rank when backend="nccl"."""
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _entry(rank, world, port, fn, args, queue, backend):
    try:
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        torch.set_num_threads(1)
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        queue.put((rank, "ok", out))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        queue.put((rank, "error", traceback.format_exc()))


def run_ranks(world, fn, *args, timeout=300, backend="gloo"):
    """fn(rank, world, *args) -> picklable; returns the list of per-rank results."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, queue, backend)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = queue.get(timeout=timeout)
            if status != "ok":
                raise RuntimeError("rank %d failed:\n%s" % (rank, payload))
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
